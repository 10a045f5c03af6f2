"""Step engine for ragged batches: every step packs whatever each live request brings — a portion of its prompt of
any length, or one decoded token — and runs it through ``ModelShard.forward`` once.

What it owns
  * per shard a ``KVCachePool`` for the attention layers (pages of ``block_size`` tokens, handed out as a request
    grows and given back at its end) and a ``RecurrentStatePool`` for the recurrent layers (one slot per live
    request);
  * the request table (tokens held, blocks, state slot) and the per-step ``RaggedBatchState`` all layers share;
  * a scheduler (``generate`` / ``batch_inference``) that admits requests while slots and pages last, feeds prompts in
    chunks beside the decoding requests' single tokens under a token budget per step, samples greedily and retires
    finished requests — the reference's ``ContinuousBatcher`` protocol (worker/batch_processor.py:302-336) with the
    batching done per step instead of per call.

``step`` is the only path to the model: ``generate`` and the trace replay tool both go through it.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .paged_layer import RaggedBatchState, RaggedLayerCache
from .worker.distributed.kv_cache import CacheBlock, KVCachePool, RecurrentStatePool
from .worker.distributed.model_shard import ModelShard


@dataclass
class _Request:
    rid: Any
    slot: int
    blocks: List[Optional[List[List[CacheBlock]]]]     # per shard: per attention layer, its blocks (None: no pool)
    length: int = 0                                    # tokens already in cache / state
    table: List[int] = field(default_factory=list)     # pool slots of its blocks


class RaggedStepEngine:
    """Runs packed steps of a model whose layers take ``RaggedLayerCache`` handles, on one CUDA device."""

    def __init__(self, shards: Sequence[ModelShard], max_tokens: int, max_seqs: int = 4, block_size: int = 16,
                 fp32_logits: bool = True):
        if not shards:
            raise ValueError("need at least one shard")
        self.shards = list(shards)
        self.device = torch.device(self.shards[0].device)
        if self.device.type != "cuda":
            raise RuntimeError("RaggedStepEngine runs on CUDA devices only (no CPU path)")
        self.dtype = self.shards[0].dtype
        self.config = self.shards[0].config
        self.block_size = block_size
        self.max_seqs = max_seqs
        self.num_blocks = (max_tokens + block_size - 1) // block_size
        self.fp32_logits = fp32_logits
        if self.dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False    # fp32 means fp32: no reduced-precision matrix mode
            torch.backends.cudnn.allow_tf32 = False
        cfg = self.config
        self.kv_pools: List[Optional[KVCachePool]] = []
        self.state_pools: List[Optional[RecurrentStatePool]] = []
        # per shard, per layer: (index in the page pool or None, index in the state pool or None); a layer whose mixer
        # runs an attention and a recurrence side by side keeps both
        self._layer_slot: List[List[Tuple[Optional[int], Optional[int]]]] = []
        for sh in self.shards:
            kv_shapes, st_shapes, where = [], [], []
            for i in range(sh.start_layer, sh.end_layer):
                kv, rs = cfg.kv_shape(i), cfg.state_shape(i)
                if kv is None and rs is None:
                    raise ValueError(f"layer {i} keeps neither pages nor a state")
                where.append((len(kv_shapes) if kv is not None else None, len(st_shapes) if rs is not None else None))
                if kv is not None:
                    kv_shapes.append(kv)
                if rs is not None:
                    st_shapes.append(rs)
            self._layer_slot.append(where)
            self.kv_pools.append(KVCachePool(num_layers=len(kv_shapes), num_heads=0, head_dim=0, block_size=block_size,
                                             max_blocks_per_layer=self.num_blocks, device=str(self.device),
                                             dtype=self.dtype, layer_shapes=kv_shapes) if kv_shapes else None)
            self.state_pools.append(RecurrentStatePool(st_shapes, max_seqs, device=str(self.device)) if st_shapes else None)
        self._slots = list(range(max_seqs - 1, -1, -1))
        self.requests: Dict[Any, _Request] = {}
        self._head_f32: Optional[torch.Tensor] = None
        self.layer_trace: Optional[list] = None   # set to a list: every step appends the residual after each layer

    # ---- requests ------------------------------------------------------------------------------------------------
    @property
    def free_blocks(self) -> int:
        pools = [p for p in self.kv_pools if p is not None]
        return min(len(p.layer(0)._free_blocks) for p in pools) if pools else 1 << 30

    @property
    def free_slots(self) -> int:
        return len(self._slots)

    def admit(self, rid: Any) -> _Request:
        if rid in self.requests:
            raise ValueError(f"request {rid!r} is already live")
        if not self._slots:
            raise RuntimeError("no free sequence slot")
        slot = self._slots.pop()
        for sp in self.state_pools:
            if sp is not None and sp.allocate() != slot:
                raise RuntimeError("state pools disagree on slot numbers")
        req = _Request(rid, slot, [p.allocate_sequence(0) if p is not None else None for p in self.kv_pools])
        self.requests[rid] = req
        return req

    def finish(self, rid: Any) -> None:
        req = self.requests.pop(rid)
        for pool, blocks in zip(self.kv_pools, req.blocks):
            if pool is not None:
                for li, layer_blocks in enumerate(blocks):
                    pool.layer(li).unpin(b.block_id for b in layer_blocks)
                pool.free_sequence(blocks)
        for sp in self.state_pools:
            if sp is not None:
                sp.free(req.slot)
        self._slots.append(req.slot)

    def release(self) -> None:
        for rid in list(self.requests):
            self.finish(rid)

    def _grow(self, req: _Request, new_len: int) -> None:
        have = len(req.table)
        need = (new_len + self.block_size - 1) // self.block_size
        if need <= have:
            return
        if need - have > self.free_blocks:
            raise RuntimeError(f"KV pages exhausted: request needs {need - have} more, {self.free_blocks} free")
        row = None
        for pool, blocks in zip(self.kv_pools, req.blocks):
            if pool is None:
                continue
            pool.extend_sequence(blocks, new_len)
            for li, layer_blocks in enumerate(blocks):
                pool.layer(li).pin(b.block_id for b in layer_blocks[have:])   # a live request's pages are not evictable
                got = [b.slot for b in layer_blocks[have:]]
                if row is None:
                    row = got
                elif got != row:
                    raise RuntimeError("layers disagree on block slots; per-layer tables are not supported here")
        if row is None:   # a model without attention layers keeps no pages
            row = [0] * (need - have)
        req.table.extend(row)

    # ---- the step ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: Sequence[Tuple[Any, Sequence[int], Sequence[int]]]) -> Optional[torch.Tensor]:
        """One packed step.  ``entries``: ``(request id, its next tokens, indices among them whose logits are
        wanted)``; unknown ids are admitted.  Returns fp32 logits ``[wanted, vocab]`` on the device in the order of
        the entries and their indices, or None when nothing was wanted."""
        bs = self.block_size
        ids: List[int] = []
        pos_l: List[np.ndarray] = []
        slot_l: List[np.ndarray] = []
        spans, scans, wanted, rows = [], [], [], []
        # refuse the whole step before touching anything when its pages or slots do not fit
        new_blocks, new_seqs, seen = 0, 0, set()
        for rid, toks, _want in entries:
            if len(toks) == 0:
                continue
            if rid in seen:
                raise ValueError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            req = self.requests.get(rid)
            have, length = (len(req.table), req.length) if req is not None else (0, 0)
            new_seqs += req is None
            new_blocks += max(0, (length + len(toks) + bs - 1) // bs - have)
        if new_seqs > self.free_slots:
            raise RuntimeError(f"no free sequence slot: the step admits {new_seqs}, {self.free_slots} free")
        if new_blocks > self.free_blocks:
            raise RuntimeError(f"KV pages exhausted: the step needs {new_blocks} more, {self.free_blocks} free")
        for rid, toks, want in entries:
            n = len(toks)
            if n == 0:
                continue
            req = self.requests.get(rid) or self.admit(rid)
            self._grow(req, req.length + n)
            p = np.arange(req.length, req.length + n, dtype=np.int64)
            table = np.asarray(req.table, dtype=np.int64)
            pos_l.append(p)
            slot_l.append(table[p // bs] * bs + p % bs)
            first = len(ids)
            spans.append((first, n, len(rows), req.length))
            scans.append((first, n, req.slot, 1 if req.length == 0 else 0))
            wanted.extend(first + int(w) for w in want)
            rows.append(req.table)
            ids.extend(int(t) for t in toks)
            req.length += n
        if not ids:
            return None
        dev = self.device
        width = max(len(r) for r in rows)
        tables = np.zeros((len(rows), max(width, 1)), dtype=np.int32)
        for b, r in enumerate(rows):
            tables[b, :len(r)] = r

        def up(a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(dev, non_blocking=True)

        st = RaggedBatchState(
            tok_pos=up(np.concatenate(pos_l).astype(np.int32)),
            slot_mapping=up(np.concatenate(slot_l)),
            block_tables=up(tables),
            scan_seqs=up(np.asarray(scans, dtype=np.int32)),
            spans=spans,
            tok_row=up(np.repeat(np.arange(len(spans), dtype=np.int32), [sp[1] for sp in spans])),
            scan_host=scans,
        )
        h = up(np.asarray(ids, dtype=np.int64))
        st.token_ids = h
        for si, shard in enumerate(self.shards):
            handles = []
            for kv_j, st_j in self._layer_slot[si]:
                c = self.kv_pools[si].layer(kv_j) if kv_j is not None else None
                handles.append(RaggedLayerCache(c.key_pool if c is not None else None,
                                                c.value_pool if c is not None else None,
                                                self.state_pools[si].layer(st_j) if st_j is not None else None, st))
            if self.layer_trace is not None:
                h = self._forward_traced(shard, h, handles)
            else:
                h, _ = shard.forward(h, past_key_values=handles, use_cache=True)
        if not wanted:
            return None
        sel = h.index_select(0, torch.tensor(wanted, dtype=torch.int64, device=dev))
        return self._logits(sel)

    def _forward_traced(self, shard: ModelShard, h: torch.Tensor, handles) -> torch.Tensor:
        """``shard.forward`` unrolled so that the residual stream after every layer can be recorded."""
        if shard.is_first_shard and hasattr(shard, "embed_tokens"):
            h = shard.embed_tokens(h)
        for layer, handle in zip(shard.layers, handles):
            h = layer(h, past_key_value=handle, use_cache=True)[0]
            self.layer_trace.append(h.clone())
        if shard.is_last_shard and getattr(shard, "norm", None) is not None:
            h = shard.norm(h)
        return h

    def _logits(self, rows: torch.Tensor) -> torch.Tensor:
        last = self.shards[-1]
        if not self.fp32_logits or self.dtype == torch.float32:
            return last.get_logits(rows).to(torch.float32)
        if self._head_f32 is None:   # fp32 accumulation AND fp32 output of the storage-dtype operands
            self._head_f32 = last.lm_head.weight.detach().to(torch.float32)
        return F.linear(rows.to(torch.float32), self._head_f32)

    # ---- scheduler -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, prefill_chunk: int = 512,
                 token_budget: int = 4096, eos_token_id: Optional[int] = None) -> List[List[int]]:
        """Greedy generation for any number of prompts with continuous batching: up to ``max_seqs`` requests are
        live; each step carries one token of every decoding request plus prompt chunks (``prefill_chunk`` tokens at
        most per request) while the step's ``token_budget`` lasts.  A request is admitted when a slot is free and the
        pages for its prompt and its new tokens are not promised to the live ones.  Returns the new tokens in the
        callers' order."""
        from . import ops

        bs = self.block_size
        out: List[List[int]] = [[] for _ in prompts]
        if max_new_tokens <= 0:
            return out
        need_blocks = [(len(p) + max_new_tokens + bs - 1) // bs for p in prompts]
        for i, p in enumerate(prompts):
            if len(p) < 1:
                raise ValueError("empty prompt")
            if need_blocks[i] > self.num_blocks and any(pool is not None for pool in self.kv_pools):
                raise ValueError(f"prompt {i} with its new tokens needs {need_blocks[i]} pages, the pool has {self.num_blocks}")
        waiting = deque(range(len(prompts)))
        live: Dict[int, Dict[str, Any]] = {}
        promised = 0
        base = len(self.requests)
        while waiting or live:
            while waiting and self.free_slots > 0 and promised + need_blocks[waiting[0]] <= self.num_blocks - base:
                i = waiting.popleft()
                promised += need_blocks[i]
                live[i] = {"fed": 0, "next": None}
                self.admit(("gen", id(out), i))
            if not live:
                raise RuntimeError("nothing can be admitted: the pool is held by other requests")
            budget = token_budget
            entries, owners = [], []
            for i, s in live.items():        # decoding requests first: one token each
                if s["next"] is not None:
                    entries.append((("gen", id(out), i), [s["next"]], [0]))
                    owners.append(i)
                    budget -= 1
            for i, s in live.items():        # then prompt chunks while the budget lasts
                if s["next"] is None and budget > 0:
                    n = min(prefill_chunk, len(prompts[i]) - s["fed"], budget)
                    chunk = list(prompts[i][s["fed"]:s["fed"] + n])
                    s["fed"] += n
                    budget -= n
                    done = s["fed"] == len(prompts[i])
                    entries.append((("gen", id(out), i), chunk, [n - 1] if done else []))
                    if done:
                        owners.append(i)
            logits = self.step(entries)
            if logits is None:
                continue
            toks = ops.argmax_rows(logits).tolist()
            for i, tok in zip(owners, toks):
                out[i].append(tok)
                live[i]["next"] = tok
                if len(out[i]) >= max_new_tokens or (eos_token_id is not None and tok == eos_token_id):
                    self.finish(("gen", id(out), i))
                    promised -= need_blocks[i]
                    del live[i]
        return out

    # ---- ContinuousBatcher protocol (reference: worker/batch_processor.py:302-336) ----------------------------------
    def batch_inference(self, params_list: List[Dict[str, Any]]) -> List[Any]:
        """One result (or Exception) per request; each carries ``input_ids`` and ``max_new_tokens``."""
        results: List[Any] = [None] * len(params_list)
        good = []
        for i, p in enumerate(params_list):
            try:
                if len(p["input_ids"]) < 1:
                    raise ValueError("empty input_ids")
                good.append(i)
            except Exception as exc:  # noqa: BLE001 - per-item failure is part of the protocol
                results[i] = exc
        if good:
            try:
                n_new = max(int(params_list[i].get("max_new_tokens", 16)) for i in good)
                rows = self.generate([params_list[i]["input_ids"] for i in good], n_new)
                for row, i in zip(rows, good):
                    want = int(params_list[i].get("max_new_tokens", 16))
                    results[i] = {"output_ids": row[:want],
                                  "usage": {"prompt_tokens": len(params_list[i]["input_ids"]), "completion_tokens": want}}
            except Exception as exc:  # noqa: BLE001
                self.release()
                for i in good:
                    results[i] = exc
        return results
