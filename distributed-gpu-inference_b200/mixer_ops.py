"""Torch-tensor front end of libb200_mixers.so (include/b200_mixers.h): ragged-batch mixers and feed-forward pieces.

Same rules as ``ops``: shapes are checked on the host, raw device pointers and torch's current stream go to the
library, nothing here computes and nothing falls back to torch.  Activations of a step are packed ``[n_tok, ...]``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .ops import DTYPE_ID, _need_cuda, _stream


# benchmark instrumentation: when set to a list, every op appends (name, start event, end event) recorded on the
# launching stream around its C-ABI call
EVENTS: Optional[list] = None


def _timed(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if EVENTS is None:
            return fn(*args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn(*args, **kwargs)
        b.record()
        EVENTS.append((fn.__name__, a, b))
        return out

    return wrapper


def _lib_():
    return _lib.load_mixers()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _rows2(x: torch.Tensor) -> int:
    """Row stride of a 2-D view whose last dimension is contiguous."""
    if x.dim() != 2 or (x.shape[1] > 1 and x.stride(1) != 1):
        raise ValueError("expected a 2-D tensor with a contiguous last dimension")
    return x.stride(0) if x.shape[0] > 1 else max(x.stride(0), x.shape[1])


@_timed
def offset_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * (1 + weight)``: fp32 ``[rows, width]`` in, the weight's dtype out."""
    _need_cuda(x, weight)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise ValueError("the residual stream is a contiguous fp32 [rows, width] tensor")
    out = torch.empty(x.shape, dtype=weight.dtype, device=x.device)
    rc = _lib_().b200_offset_rmsnorm(out.data_ptr(), x.data_ptr(), weight.data_ptr(), float(eps), x.shape[0], x.shape[1],
                                     DTYPE_ID[weight.dtype], _stream())
    _lib.check_mixers(rc, "b200_offset_rmsnorm")
    return out


@_timed
def postnorm_residual(x: torch.Tensor, y: torch.Tensor, w_post: torch.Tensor, mult: float, eps: float,
                      w_next: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """In place ``x += mult * offset_norm(y; w_post)`` (fp32); returns ``offset_norm(x; w_next)`` in the weights'
    dtype when ``w_next`` is given.  ``y``: the weights' dtype or fp32."""
    _need_cuda(x, y, w_post)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or y.shape != x.shape:
        raise ValueError("x must be contiguous fp32 [rows, width] and y of the same shape")
    if y.dtype not in (w_post.dtype, torch.float32):
        raise TypeError("y must have the weights' dtype or be fp32")
    out = torch.empty(x.shape, dtype=w_post.dtype, device=x.device) if w_next is not None else None
    rc = _lib_().b200_postnorm_residual(x.data_ptr(), y.data_ptr(), _rows2(y), int(y.dtype == torch.float32 and
                                        w_post.dtype != torch.float32), w_post.data_ptr(), float(mult), _ptr(w_next),
                                        _ptr(out), float(eps), x.shape[0], x.shape[1], DTYPE_ID[w_post.dtype], _stream())
    _lib.check_mixers(rc, "b200_postnorm_residual")
    return out


@_timed
def value_prep_append(k: torch.Tensor, v: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      slot_mapping: torch.Tensor, eps: float, v_prev: Optional[torch.Tensor] = None, lam: float = 0.0,
                      v_keep: Optional[torch.Tensor] = None) -> None:
    """Unit-RMS values per head (optionally mixed with ``v_prev``), then k / v into the pools at ``slot_mapping``.
    ``k [n, G*dk]``, ``v [n, G*dv]`` (column slices of a projection are fine); pools ``[blocks, G, bs, dk|dv]``."""
    _need_cuda(k, v, k_pool, v_pool, slot_mapping)
    nb, G, bs, dk = k_pool.shape
    dv = v_pool.shape[3]
    n = k.shape[0]
    if k.shape[1] != G * dk or v.shape != (n, G * dv) or tuple(v_pool.shape[:3]) != (nb, G, bs):
        raise ValueError("k / v do not match the pools")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != n:
        raise ValueError("slot_mapping must be int64 [n_tok]")
    for t in (v_prev, v_keep):
        if t is not None and (tuple(t.shape) != (n, G * dv) or not t.is_contiguous() or t.dtype != v.dtype):
            raise ValueError("v_prev / v_keep must be contiguous [n_tok, G*dv] in the storage dtype")
    rc = _lib_().b200_value_prep_append(k.data_ptr(), _rows2(k), v.data_ptr(), _rows2(v), _ptr(v_prev), _ptr(v_keep),
                                        float(lam), float(eps), k_pool.data_ptr(), v_pool.data_ptr(),
                                        slot_mapping.data_ptr(), n, G, dk, dv, bs, nb, DTYPE_ID[k_pool.dtype], _stream())
    _lib.check_mixers(rc, "b200_value_prep_append")


def attn_tile_tokens(n_tokens: int, H: int, G: int) -> int:
    return int(_lib_().b200_biased_attn_tile_tokens(int(n_tokens), H, G))


@_timed
def biased_paged_attention(q: torch.Tensor, gate: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: torch.Tensor,
                           block_tables: torch.Tensor, tiles: torch.Tensor, max_tile_tokens: int, tok_pos: torch.Tensor,
                           bias_lut: torch.Tensor, scale: float, temp_coef: float, temp_every: int, H: int,
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of packed rows ``q [n, H*dk]`` over the paged cache with a distance-bias table
    ``bias_lut [H, L]`` (fp32), a query temperature and a sigmoid gate ``gate [n, H]``; returns ``[n, H*dv]``
    (the tiles' rows of ``out`` when given)."""
    _need_cuda(q, k_pool, v_pool, block_tables, tiles, tok_pos, bias_lut)
    nb, G, bs, dk = k_pool.shape
    dv = v_pool.shape[3]
    n = q.shape[0]
    if q.shape[1] != H * dk or (gate is not None and tuple(gate.shape) != (n, H)):
        raise ValueError("q / gate do not match the head layout")
    if block_tables.dtype != torch.int32 or tiles.dtype != torch.int32 or tok_pos.dtype != torch.int32:
        raise TypeError("block tables, tiles and positions are int32")
    if tiles.dim() != 2 or tiles.shape[1] != 3 or not tiles.is_contiguous():
        raise ValueError("tiles must be contiguous int32 [n_tiles, 3]")
    if bias_lut.dtype != torch.float32 or bias_lut.shape[0] != H or not bias_lut.is_contiguous():
        raise ValueError("bias_lut must be contiguous fp32 [H, L]")
    if out is None:
        out = torch.empty((n, H * dv), dtype=q.dtype, device=q.device)
    rc = _lib_().b200_biased_paged_attn(out.data_ptr(), q.data_ptr(), _rows2(q), _ptr(gate),
                                        _rows2(gate) if gate is not None else 0, k_pool.data_ptr(), v_pool.data_ptr(),
                                        block_tables.data_ptr(), block_tables.stride(0), tiles.data_ptr(), tiles.shape[0],
                                        int(max_tile_tokens), tok_pos.data_ptr(), bias_lut.data_ptr(), bias_lut.shape[1],
                                        float(scale), float(temp_coef), int(temp_every), H, G, dk, dv, bs,
                                        DTYPE_ID[q.dtype], _stream())
    _lib.check_mixers(rc, "b200_biased_paged_attn")
    return out


def prompt_tile_tokens(H: int, G: int) -> int:
    """Tokens of one sequence a CTA of the tensor-core kernel serves: 64 rows over the heads of a kv group."""
    return int(_lib_().b200_biased_prompt_attn_tile_tokens(int(H), int(G)))


def prompt_attention_supported(dk: int, dv: int, dtype: torch.dtype) -> bool:
    return bool(_lib_().b200_biased_prompt_attn_supported(int(dk), int(dv), DTYPE_ID[dtype]))


@_timed
def biased_prompt_attention(out: torch.Tensor, q: torch.Tensor, gate: Optional[torch.Tensor], k_pool: torch.Tensor,
                            v_pool: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor, tok_pos: torch.Tensor,
                            bias_lut: torch.Tensor, scale: float, temp_coef: float, temp_every: int, H: int,
                            max_tile_tokens: int = 0) -> None:
    """``biased_paged_attention`` on the tensor cores, for prompt portions and decoded tokens alike; writes the tiles'
    rows of ``out`` ``[n, H*dv]`` (16-bit dtypes, see ``prompt_attention_supported``).  ``tiles``: up to
    ``prompt_tile_tokens(H, G)`` tokens each; ``max_tile_tokens``: the largest tile (0 = unknown) — steps of decoded
    tokens only take the variant whose warps split the keys."""
    _need_cuda(out, q, k_pool, v_pool, block_tables, tiles, tok_pos, bias_lut)
    nb, G, bs, dk = k_pool.shape
    dv = v_pool.shape[3]
    n = q.shape[0]
    if q.shape[1] != H * dk or tuple(out.shape) != (n, H * dv) or not out.is_contiguous() or out.dtype != q.dtype:
        raise ValueError("q / out do not match the head layout")
    if gate is not None and tuple(gate.shape) != (n, H):
        raise ValueError("gate must be [n, H]")
    if tiles.dtype != torch.int32 or tiles.dim() != 2 or tiles.shape[1] != 3 or not tiles.is_contiguous():
        raise ValueError("tiles must be contiguous int32 [n_tiles, 3]")
    if bias_lut.dtype != torch.float32 or bias_lut.shape[0] != H or not bias_lut.is_contiguous():
        raise ValueError("bias_lut must be contiguous fp32 [H, L]")
    rc = _lib_().b200_biased_prompt_attn(out.data_ptr(), q.data_ptr(), _rows2(q), _ptr(gate),
                                         _rows2(gate) if gate is not None else 0, k_pool.data_ptr(), v_pool.data_ptr(),
                                         block_tables.data_ptr(), block_tables.stride(0), tiles.data_ptr(), tiles.shape[0],
                                         int(max_tile_tokens), tok_pos.data_ptr(), bias_lut.data_ptr(), bias_lut.shape[1], float(scale),
                                         float(temp_coef), int(temp_every), H, G, dk, dv, bs, DTYPE_ID[q.dtype], _stream())
    _lib.check_mixers(rc, "b200_biased_prompt_attn")


@_timed
def gated_scan(zq: torch.Tensor, zf: torch.Tensor, v: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor,
               state: torch.Tensor, seqs: torch.Tensor, H: int, max_count: int = 1 << 20) -> torch.Tensor:
    """Gated linear recurrence over each sequence's tokens; ``state`` fp32 ``[slots, H, dk, dv]`` is read (unless the
    sequence is fresh) and written back.  ``zq / zf [n, H*dk]``, ``v [n, H*dv]`` are column slices of ONE projection
    (same row stride).  ``max_count``: the largest token count in ``seqs`` (picks the kernel; a hint, not a bound).
    Returns the raw read-outs, fp32 ``[n, H, dv]``."""
    _need_cuda(zq, zf, v, state, seqs)
    n = zq.shape[0]
    _, Hs, dk, dv = state.shape
    if Hs != H or zq.shape[1] != H * dk or zf.shape != zq.shape or v.shape != (n, H * dv):
        raise ValueError("projections do not match the state's shape")
    stride = _rows2(zq)
    if n > 1 and (zf.stride(0) != stride or v.stride(0) != stride):
        raise ValueError("zq, zf and v must share a row stride")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise TypeError("the recurrent state is contiguous fp32")
    if seqs.dtype != torch.int32 or seqs.dim() != 2 or seqs.shape[1] != 4 or not seqs.is_contiguous():
        raise ValueError("seqs must be contiguous int32 [n_seqs, 4]")
    o = torch.empty((n, H, dv), dtype=torch.float32, device=zq.device)
    rc = _lib_().b200_gated_scan(o.data_ptr(), zq.data_ptr(), zf.data_ptr(), v.data_ptr(), stride, f_bias.data_ptr(),
                                 lower.data_ptr(), state.data_ptr(), seqs.data_ptr(), seqs.shape[0], int(max_count), H, dk, dv,
                                 DTYPE_ID[zq.dtype], _stream())
    _lib.check_mixers(rc, "b200_gated_scan")
    return o


@_timed
def head_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 ``[..., dv]`` rows -> ``x * rsqrt(mean(x^2) + eps) * weight`` in the weight's dtype."""
    _need_cuda(x, weight)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32")
    dv = x.shape[-1]
    out = torch.empty(x.shape, dtype=weight.dtype, device=x.device)
    rc = _lib_().b200_head_rmsnorm(out.data_ptr(), x.data_ptr(), weight.data_ptr(), float(eps), x.numel() // dv, dv,
                                   DTYPE_ID[weight.dtype], _stream())
    _lib.check_mixers(rc, "b200_head_rmsnorm")
    return out


@_timed
def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    _need_cuda(z, coef)
    out = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    rc = _lib_().b200_polynorm(out.data_ptr(), z.data_ptr(), _rows2(z), coef.data_ptr(), float(eps), z.shape[0],
                               z.shape[1], DTYPE_ID[z.dtype], _stream())
    _lib.check_mixers(rc, "b200_polynorm")
    return out


@_timed
def sigmoid_topk(logits: torch.Tensor, top: int):
    """fp32 ``[n, E]`` logits -> ``(ids int32 [n, top], weights fp32 [n, top])``; weights are sigmoid(logit)."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise ValueError("router logits are contiguous fp32 [n, E]")
    n, E = logits.shape
    ids = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    rc = _lib_().b200_sigmoid_topk(ids.data_ptr(), w.data_ptr(), logits.data_ptr(), n, E, int(top), _stream())
    _lib.check_mixers(rc, "b200_sigmoid_topk")
    return ids, w


@_timed
def scaled_gather(h: torch.Tensor, weights: torch.Tensor, src: torch.Tensor, top: int) -> torch.Tensor:
    _need_cuda(h, weights, src)
    if not h.is_contiguous() or src.dtype != torch.int64 or weights.dtype != torch.float32:
        raise ValueError("h contiguous, src int64, weights fp32")
    xs = torch.empty((src.numel(), h.shape[1]), dtype=h.dtype, device=h.device)
    rc = _lib_().b200_scaled_gather(xs.data_ptr(), h.data_ptr(), weights.data_ptr(), src.data_ptr(), src.numel(), int(top),
                                    h.shape[1], DTYPE_ID[h.dtype], _stream())
    _lib.check_mixers(rc, "b200_scaled_gather")
    return xs


def grouped_linear_supported(K: int, dtype: torch.dtype) -> bool:
    return bool(_lib_().b200_grouped_linear_supported(int(K), DTYPE_ID[dtype]))


@_timed
def grouped_linear(xs: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """``out[r] = xs[r] @ w[e].T`` for ``offsets[e] <= r < offsets[e + 1]``: ``xs [rows, K]`` sorted by expert,
    ``w [E, N, K]``, ``offsets`` int32 ``[E + 1]`` on the device (no host copy).  16-bit dtypes."""
    _need_cuda(xs, w, offsets)
    E, N, K = w.shape
    if xs.dim() != 2 or xs.shape[1] != K or not xs.is_contiguous() or not w.is_contiguous() or xs.dtype != w.dtype:
        raise ValueError("xs [rows, K] and w [E, N, K] must be contiguous and of one dtype")
    if offsets.dtype != torch.int32 or offsets.numel() != E + 1 or not offsets.is_contiguous():
        raise ValueError("offsets must be contiguous int32 [E + 1]")
    out = torch.empty((xs.shape[0], N), dtype=xs.dtype, device=xs.device)
    rc = _lib_().b200_grouped_linear(out.data_ptr(), xs.data_ptr(), w.data_ptr(), offsets.data_ptr(), xs.shape[0], E, N, K,
                                     DTYPE_ID[xs.dtype], _stream())
    _lib.check_mixers(rc, "b200_grouped_linear")
    return out


@_timed
def clamped_glu(gu: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    _need_cuda(gu)
    if not gu.is_contiguous() or gu.shape[1] % 2:
        raise ValueError("gu must be contiguous [rows, 2*ff]")
    ff = gu.shape[1] // 2
    y = torch.empty((gu.shape[0], ff), dtype=gu.dtype, device=gu.device)
    rc = _lib_().b200_clamped_glu(y.data_ptr(), gu.data_ptr(), gu.shape[0], ff, float(limit), float(alpha),
                                  DTYPE_ID[gu.dtype], _stream())
    _lib.check_mixers(rc, "b200_clamped_glu")
    return y


@_timed
def expert_combine(ys: torch.Tensor, where: torch.Tensor, n_tok: int, top: int) -> torch.Tensor:
    _need_cuda(ys, where)
    if not ys.is_contiguous() or where.dtype != torch.int64 or where.numel() != n_tok * top:
        raise ValueError("ys contiguous, where int64 [n_tok * top]")
    out = torch.empty((n_tok, ys.shape[1]), dtype=torch.float32, device=ys.device)
    rc = _lib_().b200_expert_combine(out.data_ptr(), ys.data_ptr(), where.data_ptr(), n_tok, int(top), ys.shape[1],
                                     DTYPE_ID[ys.dtype], _stream())
    _lib.check_mixers(rc, "b200_expert_combine")
    return out


# ---- pieces for hybrid designs (csrc/b200_hybrid_ops.cu) ---------------------------------------------------------------
@_timed
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, weight_offset: float = 0.0) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * (weight_offset + weight)`` over the last dimension of 2-D rows (fp32 or the
    weight's dtype, column slices are fine); the weight's dtype out."""
    _need_cuda(x, weight)
    if x.dtype not in (torch.float32, weight.dtype) or weight.numel() != x.shape[1]:
        raise ValueError("x must be fp32 or of the weight's dtype, [rows, width] with width = weight.numel()")
    out = torch.empty(x.shape, dtype=weight.dtype, device=x.device)
    rc = _lib_().b200_rms_norm(out.data_ptr(), out.shape[1], x.data_ptr(), _rows2(x),
                               int(x.dtype == torch.float32 and weight.dtype != torch.float32), weight.data_ptr(),
                               float(weight_offset), float(eps), x.shape[0], x.shape[1], DTYPE_ID[weight.dtype], _stream())
    _lib.check_mixers(rc, "b200_rms_norm")
    return out


@_timed
def residual_add2_norm(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], w_next: Optional[torch.Tensor],
                       eps: float, weight_offset: float = 0.0) -> Optional[torch.Tensor]:
    """In place ``x += (a + b)`` on the fp32 residual (``b`` may be None); returns ``rms_norm(x; w_next)`` in the
    branches' dtype when ``w_next`` is given."""
    _need_cuda(x, a)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or a.shape != x.shape:
        raise ValueError("x must be contiguous fp32 [rows, width] and the branches of the same shape")
    if b is not None and (b.shape != x.shape or b.dtype != a.dtype):
        raise ValueError("both branches must have one shape and dtype")
    out = torch.empty(x.shape, dtype=a.dtype, device=x.device) if w_next is not None else None
    rc = _lib_().b200_residual_add2_norm(x.data_ptr(), a.data_ptr(), _rows2(a), _ptr(b), _rows2(b) if b is not None else 0,
                                         _ptr(w_next), float(weight_offset), _ptr(out), float(eps), x.shape[0], x.shape[1],
                                         DTYPE_ID[a.dtype], _stream())
    _lib.check_mixers(rc, "b200_residual_add2_norm")
    return out


@_timed
def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """``z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2`` with ``pq = (p, q)``."""
    _need_cuda(z, pq)
    if pq.numel() != 2 or pq.dtype != z.dtype:
        raise ValueError("pq holds the two numbers (p, q) in the activations' dtype")
    out = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    rc = _lib_().b200_xielu(out.data_ptr(), z.data_ptr(), _rows2(z), pq.data_ptr(), z.shape[0], z.shape[1],
                            DTYPE_ID[z.dtype], _stream())
    _lib.check_mixers(rc, "b200_xielu")
    return out


@_timed
def rotary_kv_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     slot_mapping: torch.Tensor, tok_pos: torch.Tensor, H: int, rot_dims: int, rot_base: float,
                     rotate_values: bool, interleaved: bool = False, want_table: bool = False) -> Optional[torch.Tensor]:
    """Rotary positions on q (in place) and k over their first ``rot_dims`` dimensions, optionally the values turned
    over their whole width; k and v are stored in the pools at ``slot_mapping``.  With ``want_table`` returns fp32
    ``[n, dv // 2, 2]`` = (cos, sin) of the value pairs' angles (what ``mixed_prompt_attention`` turns outputs back
    with)."""
    _need_cuda(q, k, v, k_pool, v_pool, slot_mapping, tok_pos)
    nb, G, bs, dk = k_pool.shape
    dv = v_pool.shape[3]
    n = q.shape[0]
    if q.shape[1] != H * dk or k.shape != (n, G * dk) or v.shape != (n, G * dv):
        raise ValueError("q / k / v do not match the pools")
    if slot_mapping.dtype != torch.int64 or tok_pos.dtype != torch.int32:
        raise TypeError("slot_mapping is int64, tok_pos int32")
    table = (torch.empty((n, dv // 2, 2), dtype=torch.float32, device=q.device)
             if want_table and rotate_values else None)
    rc = _lib_().b200_rotary_kv_append(q.data_ptr(), _rows2(q), k.data_ptr(), _rows2(k), v.data_ptr(), _rows2(v),
                                       k_pool.data_ptr(), v_pool.data_ptr(), slot_mapping.data_ptr(), tok_pos.data_ptr(),
                                       n, H, G, dk, dv, int(rot_dims), float(rot_base), int(rotate_values),
                                       int(interleaved), bs, nb, _ptr(table), DTYPE_ID[k_pool.dtype], _stream())
    _lib.check_mixers(rc, "b200_rotary_kv_append")
    return table


@_timed
def norm_append(x: torch.Tensor, weight: torch.Tensor, eps: float, pool: torch.Tensor, slot_mapping: torch.Tensor,
                weight_offset: float = 0.0) -> None:
    """``pool[slot] = rms_norm(x[n]; weight)``: latent rows into a one-head pool ``[blocks, 1, bs, width]``."""
    _need_cuda(x, weight, pool, slot_mapping)
    if pool.shape[1] != 1 or pool.shape[3] != x.shape[1] or x.dtype != pool.dtype or slot_mapping.dtype != torch.int64:
        raise ValueError("the pool must be [blocks, 1, block size, width] in the rows' dtype; slots int64")
    rc = _lib_().b200_norm_append(x.data_ptr(), _rows2(x), weight.data_ptr(), float(weight_offset), float(eps),
                                  pool.data_ptr(), slot_mapping.data_ptr(), x.shape[0], x.shape[1], DTYPE_ID[x.dtype],
                                  _stream())
    _lib.check_mixers(rc, "b200_norm_append")


def _value_layout(k_pool: torch.Tensor, v_pool: torch.Tensor, value_width: Optional[int], value_div: int):
    """``(value size, elements between value rows)`` of an attention call, after checking the pools against each other."""
    if v_pool.dim() != 4 or v_pool.shape[0] != k_pool.shape[0] or v_pool.shape[2] != k_pool.shape[2]:
        raise ValueError("the pools must agree on blocks and block size")
    if value_div < 1 or v_pool.shape[1] * value_div != k_pool.shape[1]:
        raise ValueError("v_pool holds one head per `value_div` key heads")
    v_row = v_pool.shape[3]
    dv = v_row if value_width is None else int(value_width)
    if dv < 1 or dv > v_row:
        raise ValueError("value_width exceeds the rows of v_pool")
    return dv, v_row


@_timed
def mixed_paged_attention(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                          block_tables: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor, scale: float,
                          talk: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, window: int = 0,
                          keep_first: int = 0, unrotate_base: Optional[float] = None, interleaved: bool = False,
                          gate: Optional[torch.Tensor] = None, softcap: float = 0.0, chunk: int = 0,
                          value_width: Optional[int] = None, value_div: int = 1) -> None:
    """Softmax attention of packed query rows over the paged cache.  ``q`` and ``out`` are 3-D ``[n, H, dk | dv]``
    VIEWS with a contiguous last dimension (any token / head strides); ``talk`` fp32 ``[H, H]`` mixes the heads'
    scores before the softmax, ``sink`` fp32 ``[H]`` adds exp(sink) to the denominator, ``window`` > 0 limits a
    position to its last ``window`` tokens plus the sequence's first ``keep_first``, ``unrotate_base`` turns the
    output back by the position over the value width, ``gate`` ``[n, H]`` is a sigmoid gate per head, ``softcap`` > 0
    bounds the scores by ``softcap * tanh(score / softcap)`` before the mask, ``chunk`` > 0 lets a position see only
    the keys of its own block of ``chunk`` positions, ``value_width`` says that the values are the first that many
    columns of the (wider) rows of ``v_pool``, ``value_div`` that ``v_pool`` holds one value head per that many key
    heads (several score maps over the same values).  ``out`` may be fp32 whatever the storage dtype (results that are
    combined before they are rounded; not with ``unrotate_base``)."""
    _need_cuda(out, q, k_pool, v_pool, block_tables, tok_row, tok_pos)
    nb, G, bs, dk = k_pool.shape
    dv, v_row = _value_layout(k_pool, v_pool, value_width, value_div)
    n, H = q.shape[0], q.shape[1]
    if q.dim() != 3 or q.shape[2] != dk or tuple(out.shape) != (n, H, dv) or q.stride(2) != 1 or out.stride(2) != 1:
        raise ValueError("q must be [n, H, dk] and out [n, H, dv] with contiguous last dimensions")
    if out.dtype not in (q.dtype, torch.float32) or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        raise TypeError("q and the pools share one dtype; out has it too, or is fp32")
    out_f32 = int(out.dtype == torch.float32 and q.dtype != torch.float32)
    for t in (block_tables, tok_row, tok_pos):
        if t.dtype != torch.int32:
            raise TypeError("block tables, token rows and positions are int32")
    for t, shape in ((talk, (H, H)), (sink, (H,))):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise ValueError("talk is contiguous fp32 [H, H], sink fp32 [H]")
    if gate is not None and (tuple(gate.shape) != (n, H) or gate.dtype != q.dtype):
        raise ValueError("gate must be [n, H] in the activations' dtype")
    rc = _lib_().b200_mixed_paged_attn_ext(out.data_ptr(), out.stride(0), out.stride(1), q.data_ptr(), q.stride(0),
                                           q.stride(1), _ptr(gate), _rows2(gate) if gate is not None else 0,
                                           k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
                                           block_tables.stride(0), tok_row.data_ptr(), tok_pos.data_ptr(), n, _ptr(talk),
                                           _ptr(sink), float(scale), float(softcap), int(window), int(keep_first),
                                           int(chunk), int(unrotate_base is not None), int(interleaved),
                                           float(unrotate_base or 0.0), H, G, dk, dv, v_row, int(value_div), out_f32, bs,
                                           DTYPE_ID[q.dtype], _stream())
    _lib.check_mixers(rc, "b200_mixed_paged_attn")


def mixed_prompt_attention_supported(H: int, G: int, dk: int, dv: int, has_talk: bool, same_pool: bool, unrotate: bool,
                                     dtype: torch.dtype) -> bool:
    return bool(_lib_().b200_mixed_prompt_attn_supported(int(H), int(G), int(dk), int(dv), int(has_talk), int(same_pool),
                                                         int(unrotate), DTYPE_ID[dtype]))


PROMPT_TILE_TOKENS = 16     # tokens of one sequence a CTA of ``mixed_prompt_attention`` serves


@_timed
def mixed_prompt_attention(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                           block_tables: torch.Tensor, tiles: torch.Tensor, tok_pos: torch.Tensor, scale: float,
                           talk: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, window: int = 0,
                           keep_first: int = 0, value_rot: Optional[torch.Tensor] = None, interleaved: bool = False,
                           gate: Optional[torch.Tensor] = None, max_context: int = 0, softcap: float = 0.0,
                           chunk: int = 0, value_width: Optional[int] = None, value_div: int = 1,
                           heads_as_rows: bool = False) -> None:
    """``mixed_paged_attention`` on the tensor cores for prompt portions and decoded tokens alike (16-bit dtypes, see
    ``mixed_prompt_attention_supported``).  ``tiles`` int32 ``[n_tiles, 3]``: up to ``PROMPT_TILE_TOKENS`` consecutive
    tokens of one sequence each, together covering every row of ``q``; ``value_rot``: the table ``rotary_kv_append``
    returned for this step's tokens; ``max_context``: the longest context of the step (a hint: steps of few tokens over
    long contexts divide the keys over several CTAs and merge); ``chunk``, ``value_width`` and ``value_div`` as in
    ``mixed_paged_attention``.  ``heads_as_rows`` (steps of single tokens over one kv head, no talk / gate / value_rot):
    the 16 rows of a tensor-core tile are 16 query heads of one token instead of 16 tokens of one head."""
    _need_cuda(out, q, k_pool, v_pool, block_tables, tiles, tok_pos)
    nb, G, bs, dk = k_pool.shape
    dv, v_row = _value_layout(k_pool, v_pool, value_width, value_div)
    n, H = q.shape[0], q.shape[1]
    if q.dim() != 3 or q.shape[2] != dk or tuple(out.shape) != (n, H, dv) or q.stride(2) != 1 or out.stride(2) != 1:
        raise ValueError("q must be [n, H, dk] and out [n, H, dv] with contiguous last dimensions")
    if out.dtype not in (q.dtype, torch.float32) or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        raise TypeError("q and the pools share one dtype; out has it too, or is fp32")
    out_f32 = int(out.dtype == torch.float32 and q.dtype != torch.float32)
    if tiles.dtype != torch.int32 or tiles.dim() != 2 or tiles.shape[1] != 3 or not tiles.is_contiguous():
        raise ValueError("tiles must be contiguous int32 [n_tiles, 3]")
    for t, shape in ((talk, (H, H)), (sink, (H,))):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise ValueError("talk is contiguous fp32 [H, H], sink fp32 [H]")
    if value_rot is not None and (tuple(value_rot.shape) != (n, dv // 2, 2) or value_rot.dtype != torch.float32
                                  or not value_rot.is_contiguous()):
        raise ValueError("value_rot must be contiguous fp32 [n, dv // 2, 2]")
    if gate is not None and (tuple(gate.shape) != (n, H) or gate.dtype != q.dtype):
        raise ValueError("gate must be [n, H] in the activations' dtype")
    if heads_as_rows and (G != 1 or talk is not None or gate is not None or value_rot is not None):
        raise ValueError("heads_as_rows needs one kv head and no talk, gate or value_rot")
    lib = _lib_()
    seen = min(max_context, window + keep_first + PROMPT_TILE_TOKENS) if window > 0 else max_context
    if chunk > 0:
        seen = min(seen, chunk + PROMPT_TILE_TOKENS)
    splits = lib.b200_mixed_prompt_attn_splits(tiles.shape[0], (seen + 31) // 32, (H + 15) // 16 if heads_as_rows else H, G,
                                               dk, dv, int(talk is not None),
                                               int(k_pool.data_ptr() == v_pool.data_ptr()), int(value_rot is not None),
                                               DTYPE_ID[q.dtype]) if max_context > 0 else 1
    ws = None
    if splits > 1:
        ws = torch.empty(lib.b200_mixed_prompt_attn_workspace(splits, n, H, dv) // 4, dtype=torch.float32, device=q.device)
    rc = lib.b200_mixed_prompt_attn_ext(out.data_ptr(), out.stride(0), out.stride(1), q.data_ptr(), q.stride(0),
                                        q.stride(1), _ptr(gate), _rows2(gate) if gate is not None else 0, k_pool.data_ptr(),
                                        v_pool.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
                                        tiles.data_ptr(), tiles.shape[0], tok_pos.data_ptr(), n, _ptr(talk), _ptr(sink),
                                        float(scale), float(softcap), int(window), int(keep_first), int(chunk),
                                        _ptr(value_rot), int(interleaved), H, G, dk, dv, v_row, int(value_div),
                                        int(heads_as_rows), out_f32, bs, int(splits), _ptr(ws), DTYPE_ID[q.dtype], _stream())
    _lib.check_mixers(rc, "b200_mixed_prompt_attn")


@_timed
def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, tail: torch.Tensor, seqs: torch.Tensor,
                     max_count: int) -> torch.Tensor:
    """Short causal convolution per channel over each sequence's tokens, then SiLU.  ``x [n, C]`` (a column slice is
    fine), ``weight [C, taps]`` (last column = the current token), ``tail`` fp32 ``[slots, taps - 1, C]`` carries each
    live sequence's last inputs between steps and is updated."""
    _need_cuda(x, weight, tail, seqs)
    C, taps = weight.shape
    if x.shape[1] != C or tail.dtype != torch.float32 or tuple(tail.shape[1:]) != (taps - 1, C) or not tail.is_contiguous():
        raise ValueError("x [n, C], weight [C, taps], tail fp32 [slots, taps - 1, C]")
    if seqs.dtype != torch.int32 or seqs.dim() != 2 or seqs.shape[1] != 4 or not seqs.is_contiguous():
        raise ValueError("seqs must be contiguous int32 [n_seqs, 4]")
    out = torch.empty((x.shape[0], C), dtype=x.dtype, device=x.device)
    rc = _lib_().b200_causal_conv_silu(out.data_ptr(), C, x.data_ptr(), _rows2(x), weight.data_ptr(), tail.data_ptr(),
                                       seqs.data_ptr(), seqs.shape[0], int(max_count), C, taps, DTYPE_ID[x.dtype], _stream())
    _lib.check_mixers(rc, "b200_causal_conv_silu")
    return out


@_timed
def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta_logit: torch.Tensor, a_logit: torch.Tensor,
               dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, seqs: torch.Tensor, G: int,
               unit_eps: float, q_scale: float) -> torch.Tensor:
    """Gated delta rule with a decay per key channel over each sequence's tokens; ``state`` fp32 ``[slots, H, dk, dv]``
    is read (unless the sequence is fresh) and written back.  ``q / k [n, G*dk]`` and ``v [n, H*dv]`` are column
    slices of ONE tensor (same row stride), ``beta_logit [n, H]``, ``a_logit [n, H*dk]``.  Returns fp32 ``[n, H, dv]``."""
    _need_cuda(q, k, v, beta_logit, a_logit, dt_bias, a_log, state, seqs)
    n = q.shape[0]
    _, H, dk, dv = state.shape
    if q.shape[1] != G * dk or k.shape != q.shape or v.shape != (n, H * dv) or beta_logit.shape != (n, H) \
            or a_logit.shape != (n, H * dk) or dt_bias.numel() != H * dk or a_log.numel() != H:
        raise ValueError("inputs do not match the state's shape")
    stride = _rows2(q)
    if n > 1 and (k.stride(0) != stride or v.stride(0) != stride):
        raise ValueError("q, k and v must share a row stride")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise TypeError("the recurrent state is contiguous fp32")
    if seqs.dtype != torch.int32 or seqs.dim() != 2 or seqs.shape[1] != 4 or not seqs.is_contiguous():
        raise ValueError("seqs must be contiguous int32 [n_seqs, 4]")
    o = torch.empty((n, H, dv), dtype=torch.float32, device=q.device)
    rc = _lib_().b200_delta_scan(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), stride, beta_logit.data_ptr(),
                                 _rows2(beta_logit), a_logit.data_ptr(), _rows2(a_logit), dt_bias.data_ptr(),
                                 a_log.data_ptr(), state.data_ptr(), seqs.data_ptr(), seqs.shape[0], H, G, dk, dv,
                                 float(unit_eps), float(q_scale), DTYPE_ID[q.dtype], _stream())
    _lib.check_mixers(rc, "b200_delta_scan")
    return o


@_timed
def head_rmsnorm_gated(x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """fp32 ``[n, H, dv]`` -> ``x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate)`` as ``[n, H*dv]`` in the weight's
    dtype; ``gate [n, H*dv]`` holds logits."""
    _need_cuda(x, weight)
    n, H, dv = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or weight.numel() != dv:
        raise ValueError("x must be contiguous fp32 [n, H, dv] and weight [dv]")
    if gate is not None and (tuple(gate.shape) != (n, H * dv) or gate.dtype != weight.dtype):
        raise ValueError("gate must be [n, H*dv] in the weight's dtype")
    out = torch.empty((n, H * dv), dtype=weight.dtype, device=x.device)
    rc = _lib_().b200_head_rmsnorm_gated(out.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(gate),
                                         _rows2(gate) if gate is not None else 0, float(eps), n, H, dv,
                                         DTYPE_ID[weight.dtype], _stream())
    _lib.check_mixers(rc, "b200_head_rmsnorm_gated")
    return out


# ---- side-by-side mixers, post-norm sublayers, grouped softmax routing (csrc/b200_parallel_ops.cu) ---------------------
def _check_seqs(seqs: torch.Tensor) -> None:
    if seqs.dtype != torch.int32 or seqs.dim() != 2 or seqs.shape[1] != 4 or not seqs.is_contiguous():
        raise ValueError("seqs must be contiguous int32 [n_seqs, 4]")


@_timed
def qknorm_rotary_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_norm: Optional[torch.Tensor],
                         k_norm: Optional[torch.Tensor], eps: float, freqs: Optional[torch.Tensor], k_pool: torch.Tensor,
                         v_pool: torch.Tensor, slot_mapping: torch.Tensor, tok_pos: torch.Tensor, H: int,
                         interleaved: bool = True) -> None:
    """Per-head RMS norm of q (in place) and k (weights ``[dk]``, None: no norm), rotary positions over the first
    ``2 * len(freqs)`` dimensions of every head with angle ``pos * freqs[i]`` (``freqs`` float64 on the device), k and v
    stored in the pools at ``slot_mapping``.  ``v_pool`` may hold fewer heads than ``k_pool`` (several score maps over the
    same values)."""
    _need_cuda(q, k, v, k_pool, v_pool, slot_mapping, tok_pos)
    nb, G, bs, dk = k_pool.shape
    Gv, dv = v_pool.shape[1], v_pool.shape[3]
    n = q.shape[0]
    if q.shape[1] != H * dk or k.shape != (n, G * dk) or v.shape != (n, Gv * dv) or v_pool.shape[0] != nb \
            or v_pool.shape[2] != bs:
        raise ValueError("q / k / v do not match the pools")
    if slot_mapping.dtype != torch.int64 or tok_pos.dtype != torch.int32:
        raise TypeError("slot_mapping is int64, tok_pos int32")
    for w in (q_norm, k_norm):
        if w is not None and (w.numel() != dk or w.dtype != q.dtype or not w.is_contiguous()):
            raise ValueError("norm weights are contiguous [dk] in the activations' dtype")
    rot_dims = 0
    if freqs is not None:
        if freqs.dtype != torch.float64 or not freqs.is_contiguous() or not freqs.is_cuda:
            raise ValueError("freqs is a contiguous float64 tensor on the device")
        rot_dims = 2 * freqs.numel()
    rc = _lib_().b200_qknorm_rotary_append_ext(q.data_ptr(), _rows2(q), k.data_ptr(), _rows2(k), v.data_ptr(), _rows2(v),
                                               _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(freqs), rot_dims,
                                               int(interleaved), k_pool.data_ptr(), v_pool.data_ptr(),
                                               slot_mapping.data_ptr(), tok_pos.data_ptr(), n, H, G, Gv, dk, dv, bs, nb,
                                               DTYPE_ID[k_pool.dtype], _stream())
    _lib.check_mixers(rc, "b200_qknorm_rotary_append")


@_timed
def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, k_scale: float,
                   state: torch.Tensor, seqs: torch.Tensor, plan=None) -> torch.Tensor:
    """Fixed-decay linear attention over each sequence's tokens: ``S <- decay[h] S + (k_scale k) v^T``, ``o = S^T q``;
    ``state`` fp32 ``[slots, H, dk, dv]`` is read (unless the sequence is fresh) and written back.  ``q / k [n, H*dk]``
    and ``v [n, H*dv]`` are column slices of ONE tensor.  Returns fp32 ``[n, H, dv]``.

    ``plan`` (``RaggedBatchState.scan_plan()``; None: every sequence runs token by token in one launch) names the long
    portions of the step as parallel segments: each segment runs as a fresh sequence against a scratch state, one launch
    chains the segments' end states into the state at every segment's start and the sequence's final state, and one adds
    what each token missed, ``decay^(t - t0 + 1) P^T q_t``.  Short sequences of the same step run as before."""
    _need_cuda(q, k, v, decay, state, seqs)
    n = q.shape[0]
    _, H, dk, dv = state.shape
    if q.shape[1] != H * dk or k.shape != q.shape or v.shape != (n, H * dv):
        raise ValueError("projections do not match the state's shape")
    stride = _rows2(q)
    if n > 1 and (k.stride(0) != stride or v.stride(0) != stride):
        raise ValueError("q, k and v must share a row stride")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise TypeError("the recurrent state is contiguous fp32")
    if decay.dtype != torch.float32 or decay.numel() != H or not decay.is_contiguous():
        raise ValueError("decay is contiguous fp32 [H]")
    _check_seqs(seqs)
    o = torch.empty((n, H, dv), dtype=torch.float32, device=q.device)
    lib, dt, st = _lib_(), DTYPE_ID[q.dtype], _stream()

    def scan(into: torch.Tensor, table: torch.Tensor) -> None:
        rc = lib.b200_retention_scan(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), stride, decay.data_ptr(),
                                     float(k_scale), into.data_ptr(), table.data_ptr(), table.shape[0], H, dk, dv, dt, st)
        _lib.check_mixers(rc, "b200_retention_scan")

    if plan is None:
        scan(state, seqs)
        return o
    if plan.direct is not None:
        scan(state, plan.direct)
    seg_state = torch.empty((plan.segs.shape[0], H, dk, dv), dtype=torch.float32, device=q.device)
    scan(seg_state, plan.segs)
    rc = lib.b200_retention_carry(state.data_ptr(), seg_state.data_ptr(), plan.parents.data_ptr(), plan.parents.shape[0],
                                  plan.segs.data_ptr(), decay.data_ptr(), H, dk, dv, st)
    _lib.check_mixers(rc, "b200_retention_carry")
    rc = lib.b200_retention_apply_carry(o.data_ptr(), q.data_ptr(), stride, seg_state.data_ptr(), plan.segs.data_ptr(),
                                        plan.segs.shape[0], decay.data_ptr(), H, dk, dv, dt, st)
    _lib.check_mixers(rc, "b200_retention_apply_carry")
    return o


@_timed
def head_norm_act_gate(x: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], eps: float,
                       dtype: torch.dtype, gate_act: str = "silu", out_scale: float = 1.0,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[n, H, dv]`` -> ``x * rsqrt(mean(x^2) + eps) [* weight] * act(gate) * out_scale`` as ``[n, H*dv]`` in
    ``dtype``; ``gate [n, H*dv]`` holds pre-activations, ``gate_act`` is ``"sigmoid"`` or ``"silu"``; ``out`` may be a
    column slice of a wider buffer."""
    _need_cuda(x)
    n, H, dv = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32 [n, H, dv]")
    if weight is not None and (weight.numel() != dv or weight.dtype != dtype):
        raise ValueError("weight must be [dv] in the output dtype")
    if gate is not None and (tuple(gate.shape) != (n, H * dv) or gate.dtype != dtype):
        raise ValueError("gate must be [n, H*dv] in the output dtype")
    if out is None:
        out = torch.empty((n, H * dv), dtype=dtype, device=x.device)
    elif tuple(out.shape) != (n, H * dv) or out.dtype != dtype:
        raise ValueError("out must be [n, H*dv] in the output dtype")
    rc = _lib_().b200_head_norm_act_gate(out.data_ptr(), _rows2(out), x.data_ptr(), _ptr(weight), _ptr(gate),
                                         _rows2(gate) if gate is not None else 0, {"sigmoid": 0, "silu": 1}[gate_act],
                                         float(out_scale), float(eps), n, H, dv, DTYPE_ID[dtype], _stream())
    _lib.check_mixers(rc, "b200_head_norm_act_gate")
    return out


@_timed
def branch_postnorm_residual(x: torch.Tensor, a: torch.Tensor, sa: float, b: Optional[torch.Tensor], sb: float,
                             w_norm: torch.Tensor, layer_scale: Optional[torch.Tensor], eps: float,
                             want_copy: bool = True) -> Optional[torch.Tensor]:
    """In place ``x += layer_scale * w_norm * y * rsqrt(mean(y^2) + eps)`` with ``y = sa a + sb b`` on the fp32 residual;
    ``a`` is fp32 or of the weights' dtype, ``b`` (optional) of the weights' dtype.  With ``want_copy`` returns the new
    ``x`` in the weights' dtype (what sublayers that read the residual itself take as GEMM input)."""
    _need_cuda(x, a, w_norm)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or a.shape != x.shape:
        raise ValueError("x must be contiguous fp32 [rows, width] and the branches of the same shape")
    T = w_norm.dtype
    if a.dtype not in (T, torch.float32) or (b is not None and (b.dtype != T or b.shape != x.shape)):
        raise TypeError("a is fp32 or of the weights' dtype, b of the weights' dtype")
    if layer_scale is not None and (layer_scale.dtype != T or layer_scale.numel() != x.shape[1]):
        raise ValueError("layer_scale must be [width] in the weights' dtype")
    out = torch.empty(x.shape, dtype=T, device=x.device) if want_copy else None
    rc = _lib_().b200_branch_postnorm_residual(x.data_ptr(), a.data_ptr(), _rows2(a), int(a.dtype == torch.float32 and
                                               T != torch.float32), float(sa), _ptr(b), _rows2(b) if b is not None else 0,
                                               float(sb), w_norm.data_ptr(), _ptr(layer_scale), _ptr(out), float(eps),
                                               x.shape[0], x.shape[1], DTYPE_ID[T], _stream())
    _lib.check_mixers(rc, "b200_branch_postnorm_residual")
    return out


@_timed
def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Contiguous fp32 tensor -> the same numbers in ``dtype``."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    rc = _lib_().b200_cast_rows(out.data_ptr(), x.data_ptr(), x.numel(), DTYPE_ID[dtype], _stream())
    _lib.check_mixers(rc, "b200_cast_rows")
    return out


@_timed
def softmax_group_topk(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int = 1,
                       keep: int = 1, sum_floor: float = 0.0):
    """fp32 ``[n, E]`` router logits -> ``(ids int32 [n, top], weights fp32 [n, top])``: softmax scores, the choice by
    score + ``correction`` inside the ``keep`` best of ``groups`` expert groups, weights = chosen scores over (their
    sum + ``sum_floor``)."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise ValueError("router logits are contiguous fp32 [n, E]")
    n, E = logits.shape
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E
                                   or not correction.is_contiguous()):
        raise ValueError("correction is contiguous fp32 [E]")
    ids = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    rc = _lib_().b200_softmax_group_topk(ids.data_ptr(), w.data_ptr(), logits.data_ptr(), _ptr(correction),
                                         float(sum_floor), n, E, int(top), int(groups), int(keep), _stream())
    _lib.check_mixers(rc, "b200_softmax_group_topk")
    return ids, w


@_timed
def gather_rows(h: torch.Tensor, src: torch.Tensor, top: int) -> torch.Tensor:
    """``xs[r] = h[src[r] // top]``: rows in expert order."""
    _need_cuda(h, src)
    if not h.is_contiguous() or src.dtype != torch.int64:
        raise ValueError("h contiguous, src int64")
    xs = torch.empty((src.numel(), h.shape[1]), dtype=h.dtype, device=h.device)
    rc = _lib_().b200_gather_rows(xs.data_ptr(), h.data_ptr(), src.data_ptr(), src.numel(), int(top), h.shape[1],
                                  DTYPE_ID[h.dtype], _stream())
    _lib.check_mixers(rc, "b200_gather_rows")
    return xs


@_timed
def weighted_expert_combine(ys: torch.Tensor, where: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                            x_self: torch.Tensor, shared: Optional[torch.Tensor], n_real: int) -> torch.Tensor:
    """fp32 ``[n, width]``: ``sum_k weights[n, k] * (ys[where[n*top + k]] if ids[n, k] < n_real else x_self[n])`` plus
    ``shared[n]`` when given.  ``x_self`` is the fp32 row an identity expert returns."""
    _need_cuda(ys, where, ids, weights, x_self)
    n, top = ids.shape
    width = x_self.shape[1]
    if not ys.is_contiguous() or ys.shape[1] != width or where.dtype != torch.int64 or where.numel() != n * top:
        raise ValueError("ys contiguous [rows, width], where int64 [n * top]")
    if ids.dtype != torch.int32 or weights.dtype != torch.float32 or not ids.is_contiguous() or not weights.is_contiguous():
        raise ValueError("ids int32 and weights fp32, contiguous [n, top]")
    if x_self.dtype != torch.float32 or not x_self.is_contiguous() or x_self.shape[0] != n:
        raise ValueError("x_self is contiguous fp32 [n, width]")
    if shared is not None and (shared.shape != x_self.shape or shared.dtype != ys.dtype or not shared.is_contiguous()):
        raise ValueError("shared rows are contiguous [n, width] in the experts' dtype")
    out = torch.empty((n, width), dtype=torch.float32, device=ys.device)
    rc = _lib_().b200_weighted_expert_combine(out.data_ptr(), ys.data_ptr(), where.data_ptr(), ids.data_ptr(),
                                              weights.data_ptr(), x_self.data_ptr(), _ptr(shared), n, top, int(n_real),
                                              width, DTYPE_ID[ys.dtype], _stream())
    _lib.check_mixers(rc, "b200_weighted_expert_combine")
    return out


# ---- token shift, sigmoid-gated post-norm sublayers, a decoupled rotated key part (csrc/b200_gated_ops.cu) -----------
@_timed
def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, seqs: torch.Tensor, max_count: int,
                want_cast: bool = False):
    """``out[t] = x[t] + (x[t - 1] - x[t]) * mu`` per channel over each sequence's tokens, in ``mu``'s dtype; the row before
    a portion comes from ``state`` fp32 ``[slots, width]`` (zero for a fresh sequence), which then receives the portion's
    last row.  Returns ``(out, x rounded to that dtype or None)``."""
    _need_cuda(x, mu, state, seqs)
    _check_seqs(seqs)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise ValueError("x must be contiguous fp32 [rows, width]")
    n, W = x.shape
    if mu.numel() != W or not mu.is_contiguous():
        raise ValueError("mu is contiguous [width]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != W or not state.is_contiguous():
        raise ValueError("state is contiguous fp32 [slots, width]")
    T = mu.dtype
    out = torch.empty((n, W), dtype=T, device=x.device)
    cast = torch.empty((n, W), dtype=T, device=x.device) if want_cast else None
    rc = _lib_().b200_token_shift(out.data_ptr(), W, _ptr(cast), x.data_ptr(), mu.data_ptr(), state.data_ptr(),
                                  seqs.data_ptr(), seqs.shape[0], int(max_count), W, DTYPE_ID[T], _stream())
    _lib.check_mixers(rc, "b200_token_shift")
    return out, cast


@_timed
def latent_rotary_append(q_rot: torch.Tensor, q_out: torch.Tensor, dkv: torch.Tensor, c_norm: torch.Tensor, eps: float,
                         freqs: Optional[torch.Tensor], gain: float, pool: torch.Tensor, slot_mapping: torch.Tensor,
                         tok_pos: torch.Tensor) -> None:
    """``dkv [n, rank + dr]``: its first ``rank = len(c_norm)`` columns RMS-normed with ``c_norm`` and its last ``dr``
    turned by the position go to one row of the one-head ``pool [blocks, 1, bs, rank + dr]``; ``q_out[n, h, :] =
    turn(q_rot[n, h, :])`` for 3-D views ``[n, H, dr]`` with contiguous last dimensions that do not overlap.  Pairs
    ``(2i, 2i + 1)``, ``i < len(freqs)``, are turned by ``pos * freqs[i]`` with cos and sin times ``gain``."""
    _need_cuda(q_rot, q_out, dkv, c_norm, pool, slot_mapping, tok_pos)
    n, H, dr = q_rot.shape
    rank = c_norm.numel()
    if q_out.shape != q_rot.shape or q_rot.stride(2) != 1 or q_out.stride(2) != 1:
        raise ValueError("q_rot and q_out are [n, H, dr] views with contiguous last dimensions")
    if dkv.shape != (n, rank + dr) or pool.dim() != 4 or pool.shape[1] != 1 or pool.shape[3] != rank + dr \
            or not pool.is_contiguous():
        raise ValueError("dkv is [n, rank + dr] and the pool [blocks, 1, block size, rank + dr]")
    T = pool.dtype
    if any(t.dtype != T for t in (q_rot, q_out, dkv, c_norm)):
        raise TypeError("activations, norm weight and pool share one dtype")
    if slot_mapping.dtype != torch.int64 or tok_pos.dtype != torch.int32:
        raise TypeError("slot_mapping is int64, tok_pos int32")
    rot_dims = 0
    if freqs is not None:
        if freqs.dtype != torch.float64 or not freqs.is_contiguous() or not freqs.is_cuda:
            raise ValueError("freqs is a contiguous float64 tensor on the device")
        rot_dims = 2 * freqs.numel()
    rc = _lib_().b200_latent_rotary_append(q_rot.data_ptr(), q_rot.stride(0), q_rot.stride(1), q_out.data_ptr(),
                                           q_out.stride(0), q_out.stride(1), dkv.data_ptr(), _rows2(dkv), c_norm.data_ptr(),
                                           float(eps), _ptr(freqs), float(gain), rot_dims, pool.data_ptr(),
                                           slot_mapping.data_ptr(), tok_pos.data_ptr(), n, H, dr, rank, DTYPE_ID[T],
                                           _stream())
    _lib.check_mixers(rc, "b200_latent_rotary_append")


@_timed
def head_diff_norm(a: torch.Tensor, lam: float, out_scale: float, eps: float, rep: int, dtype: Optional[torch.dtype] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [n, 2H, dv]`` (a view with a contiguous last dimension; fp32 or the storage dtype) holds two score maps'
    outputs per head, map 1 of head ``h`` at ``(h // rep) * 2 rep + h % rep`` and map 2 ``rep`` heads further: returns
    ``[n, H * dv]`` = ``unit_rms(a1 - lam a2) * out_scale`` per head in ``dtype`` (default: ``a``'s)."""
    _need_cuda(a)
    dtype = dtype or (out.dtype if out is not None else a.dtype)
    if a.dtype not in (dtype, torch.float32):
        raise TypeError("a is fp32 or of the output's dtype")
    n, H2, dv = a.shape
    if a.stride(2) != 1 or H2 % (2 * rep):
        raise ValueError("a is [n, 2H, dv] with a contiguous last dimension, H a multiple of rep")
    H = H2 // 2
    if out is None:
        out = torch.empty((n, H * dv), dtype=dtype, device=a.device)
    rc = _lib_().b200_head_diff_norm(out.data_ptr(), _rows2(out), a.data_ptr(), a.stride(0), a.stride(1),
                                     int(a.dtype == torch.float32 and dtype != torch.float32), float(lam), float(out_scale),
                                     float(eps), n, H, int(rep), dv, DTYPE_ID[dtype], _stream())
    _lib.check_mixers(rc, "b200_head_diff_norm")
    return out


@_timed
def gated_postnorm_residual(x: torch.Tensor, a: torch.Tensor, gate: Optional[torch.Tensor], w_norm: torch.Tensor,
                            weight_offset: float, eps: float, want_copy: bool = True) -> Optional[torch.Tensor]:
    """In place ``x += (weight_offset + w_norm) * y * rsqrt(mean(y^2) + eps)`` with ``y = a * sigmoid(gate)`` on the fp32
    residual; ``a`` is fp32 or of the weights' dtype, ``gate`` (logits, optional) of the weights' dtype.  With
    ``want_copy`` returns the new ``x`` in the weights' dtype."""
    _need_cuda(x, a, w_norm)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or a.shape != x.shape:
        raise ValueError("x must be contiguous fp32 [rows, width] and the branch of the same shape")
    T = w_norm.dtype
    if a.dtype not in (T, torch.float32) or (gate is not None and (gate.dtype != T or gate.shape != x.shape)):
        raise TypeError("a is fp32 or of the weights' dtype, the gate of the weights' dtype")
    out = torch.empty(x.shape, dtype=T, device=x.device) if want_copy else None
    rc = _lib_().b200_gated_postnorm_residual(x.data_ptr(), a.data_ptr(), _rows2(a),
                                              int(a.dtype == torch.float32 and T != torch.float32), _ptr(gate),
                                              _rows2(gate) if gate is not None else 0, w_norm.data_ptr(),
                                              float(weight_offset), _ptr(out), float(eps), x.shape[0], x.shape[1],
                                              DTYPE_ID[T], _stream())
    _lib.check_mixers(rc, "b200_gated_postnorm_residual")
    return out


@_timed
def relu_squared(z: torch.Tensor) -> torch.Tensor:
    """``max(z, 0)^2`` of 2-D rows (a column slice is fine), contiguous out."""
    _need_cuda(z)
    out = torch.empty(z.shape, dtype=z.dtype, device=z.device)
    if z.shape[0]:
        rc = _lib_().b200_relu_squared(out.data_ptr(), z.data_ptr(), _rows2(z), z.shape[0], z.shape[1], DTYPE_ID[z.dtype],
                                       _stream())
        _lib.check_mixers(rc, "b200_relu_squared")
    return out


@_timed
def gated_table_rows(z: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(z[n, c]) * table[tokens[n], col0 + c]``: ``z [n, d]``, ``table [rows, >= col0 + d]`` of the same dtype,
    ``tokens`` int64 ``[n]``."""
    _need_cuda(z, table, tokens)
    n, d = z.shape
    if table.dtype != z.dtype or table.dim() != 2 or table.stride(1) != 1 or col0 + d > table.shape[1]:
        raise ValueError("the table is 2-D in z's dtype with at least col0 + d columns")
    if tokens.dtype != torch.int64 or tokens.numel() != n or not tokens.is_contiguous():
        raise ValueError("tokens is contiguous int64 [n]")
    out = torch.empty((n, d), dtype=z.dtype, device=z.device)
    rc = _lib_().b200_gated_table_rows(out.data_ptr(), z.data_ptr(), _rows2(z), table.data_ptr(), table.stride(0), int(col0),
                                       tokens.data_ptr(), n, d, DTYPE_ID[z.dtype], _stream())
    _lib.check_mixers(rc, "b200_gated_table_rows")
    return out


@_timed
def router_logits(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``x [n, width] @ w [E, width].T + bias``: a router's logits, every sum in an order fixed by the width (a
    token's choice of experts does not depend on the rest of the step)."""
    _need_cuda(x, w)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] \
            or not x.is_contiguous() or not w.is_contiguous():
        raise ValueError("x [n, width] and w [E, width] are contiguous fp32")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.shape[0] or not bias.is_contiguous()):
        raise ValueError("bias is contiguous fp32 [E]")
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    rc = _lib_().b200_router_logits(out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), x.shape[0], w.shape[0],
                                    x.shape[1], _stream())
    _lib.check_mixers(rc, "b200_router_logits")
    return out
