"""Paged KV cache: page pool, block tables, per-sequence lengths (block size 16, GQA native).

Absent from the reference, whose cache is one dense ``[B, heads, max_seq, D]`` tensor per layer with a
single shared length (opt_prime/opt_prime/kv_cache.py:96-170).  Here every layer owns K and V pools of
``[num_pages, 16, kv_heads, head_dim]``; a sequence holds a list of page ids; the decode-attention kernel
walks the block table.  Page 0 is reserved as a scratch page for padded batch slots.  The pools may live in
peer-mapped memory so that a prefill GPU can push pages into a decode GPU's pool
(:class:`aicomp_b200.serve.pd.KVPagePusher`).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..ops import _lib, attention as attn_ops

PAGE = 16
_lib.OPTIONAL_PROTOS.update({
    "b200_paged_decode_scratch_floats": [_lib.I, _lib.I, _lib.I],
    "b200_paged_decode": [_lib.P, _lib.L, _lib.P, _lib.P, _lib.P, _lib.I, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.F, _lib.I,
                          _lib.P, _lib.L, _lib.P, _lib.P],
    "b200_paged_kv_write": [_lib.P, _lib.L, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P, _lib.I, _lib.P, _lib.P, _lib.L, _lib.P],
})
_lib.rebind()


class PageAllocator:
    """Free-list of page ids (page 0 is never handed out)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free: List[int] = list(range(num_pages - 1, 0, -1))

    def available(self) -> int:
        return len(self.free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self.free):
            raise MemoryError(f"KV cache exhausted: need {n} pages, {len(self.free)} free")
        out = [self.free.pop() for _ in range(n)]
        return out

    def release(self, pages: List[int]) -> None:
        self.free.extend(pages)


class PagedKVCache:
    """Per-stage paged cache for ``n_layers`` layers; pools are views ``[layers, 2, pages, 16, kv_heads, D]``."""

    def __init__(self, n_layers: int, kv_heads: int, head_dim: int, num_pages: int, max_seqs: int, max_blocks_per_seq: int,
                 dtype=torch.bfloat16, device=None, pool: Optional[torch.Tensor] = None, layer_offset: int = 0,
                 q_heads: Optional[int] = None):
        self.n_layers, self.kv_heads, self.head_dim = n_layers, kv_heads, head_dim
        self.num_pages, self.max_seqs, self.max_blocks = num_pages, max_seqs, max_blocks_per_seq
        self.dtype, self.device = dtype, device
        self.layer_offset = layer_offset
        self.page_elems = PAGE * kv_heads * head_dim
        shape = (n_layers, 2, num_pages, PAGE, kv_heads, head_dim)
        if pool is not None:
            self.pool = pool.view(dtype).view(shape)
        else:
            self.pool = torch.zeros(shape, dtype=dtype, device=device)
        self.alloc = PageAllocator(num_pages)
        self.block_table = torch.zeros(max_seqs, max_blocks_per_seq, dtype=torch.int32, device=device)
        self.block_table_host = torch.zeros(max_seqs, max_blocks_per_seq, dtype=torch.int32)
        self.seq_pages: Dict[int, List[int]] = {}
        self.seq_len: Dict[int, int] = {}
        self.free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        # Split-KV partials of the decode kernel.  Sized once for the worst batch: CUDA graphs record its address, so it
        # must never be reallocated afterwards.
        self._scratch: Optional[torch.Tensor] = None
        self.q_heads = q_heads or kv_heads * 8
        if device is not None and torch.device(device).type == "cuda":
            worst = max(n * self._splits_for(n) for n in range(1, max_seqs + 1) if self._splits_for(n) > 1) if max_seqs else 0
            self._scratch = torch.empty(max(1, worst) * self.q_heads * (head_dim + 2), dtype=torch.float32, device=device)

    def _splits_for(self, n: int) -> int:
        return max(1, min(16, (2 * 148 + n * self.kv_heads - 1) // (n * self.kv_heads)))

    # ---- sequence management (host side) -----------------------------------------------------
    def pages_needed(self, tokens: int) -> int:
        return (tokens + PAGE - 1) // PAGE

    def can_admit(self, tokens: int) -> bool:
        return bool(self.free_slots) and self.alloc.available() >= self.pages_needed(tokens)

    def add_sequence(self, reserve_tokens: int) -> int:
        """Reserve a slot and pages for ``reserve_tokens`` tokens; returns the slot id."""
        slot = self.free_slots.pop()
        pages = self.alloc.alloc(self.pages_needed(reserve_tokens))
        if len(pages) > self.max_blocks:
            self.alloc.release(pages)
            self.free_slots.append(slot)
            raise ValueError("sequence needs more pages than max_blocks_per_seq")
        self.seq_pages[slot] = pages
        self.seq_len[slot] = 0
        self.block_table_host[slot, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        self.block_table[slot, :len(pages)].copy_(self.block_table_host[slot, :len(pages)], non_blocking=True)
        return slot

    def ensure_capacity(self, slot: int, tokens: int) -> None:
        need = self.pages_needed(tokens) - len(self.seq_pages[slot])
        if need > 0:
            new = self.alloc.alloc(need)
            start = len(self.seq_pages[slot])
            if start + need > self.max_blocks:
                self.alloc.release(new)
                raise ValueError("sequence outgrew max_blocks_per_seq")
            self.seq_pages[slot].extend(new)
            self.block_table_host[slot, start:start + need] = torch.tensor(new, dtype=torch.int32)
            self.block_table[slot, start:start + need].copy_(self.block_table_host[slot, start:start + need], non_blocking=True)

    def free_sequence(self, slot: int) -> None:
        self.alloc.release(self.seq_pages.pop(slot))
        self.seq_len.pop(slot, None)
        self.free_slots.append(slot)

    def utilisation(self) -> float:
        return 1.0 - self.alloc.available() / max(1, self.num_pages - 1)

    # ---- device side -----------------------------------------------------------------------------
    def layer_pools(self, layer_idx: int):
        l = layer_idx - self.layer_offset
        return self.pool[l, 0], self.pool[l, 1]

    def write(self, layer_idx: int, qkv: torch.Tensor, hq: int, table: torch.Tensor, seq_idx: torch.Tensor,
              positions: torch.Tensor) -> None:
        """Store K/V of the rows of the packed ``qkv`` (after RoPE): row i goes to position ``positions[i]`` of the
        sequence whose block-table row is ``table[seq_idx[i]]``."""
        k_pool, v_pool = self.layer_pools(layer_idx)
        slots = seq_idx
        if ops.kernels_for(qkv):
            lib = _lib.require()
            rc = lib.b200_paged_kv_write(qkv.data_ptr(), qkv.stride(0), hq, self.kv_heads, self.head_dim, slots.data_ptr(),
                                         positions.data_ptr(), table.data_ptr(), table.shape[1], k_pool.data_ptr(),
                                         v_pool.data_ptr(), qkv.shape[0], _lib.stream_ptr())
            _lib.check_rc(rc, "paged_kv_write")
            ops._count()
            return
        D, hkv = self.head_dim, self.kv_heads
        k = qkv[:, hq * D:(hq + hkv) * D].view(-1, hkv, D)
        v = qkv[:, (hq + hkv) * D:].view(-1, hkv, D)
        pages = table[slots.long(), (positions // PAGE).long()].long()
        k_pool[pages, (positions % PAGE).long()] = k
        v_pool[pages, (positions % PAGE).long()] = v

    def decode_attention(self, layer_idx: int, q: torch.Tensor, hq: int, table: torch.Tensor, seq_lens: torch.Tensor,
                         scale: Optional[float] = None) -> torch.Tensor:
        """``q [n, hq*D]`` (one new token per sequence; sequence i uses block-table row ``table[i]``) -> ``[n, hq*D]``."""
        n, D = q.shape[0], self.head_dim
        scale = scale if scale is not None else D ** -0.5
        k_pool, v_pool = self.layer_pools(layer_idx)
        if ops.kernels_for(q) and D == 128:
            lib = _lib.require()
            out = torch.empty(n, hq * D, dtype=q.dtype, device=q.device)
            max_len_pages = table.shape[1]
            splits = self._splits_for(n) if n <= self.max_seqs else 1
            scratch = None
            need = lib.b200_paged_decode_scratch_floats(n, hq, splits)
            if need:
                if self._scratch is None or self._scratch.numel() < need:
                    raise RuntimeError("decode scratch too small: construct PagedKVCache with the model's q_heads")
                scratch = self._scratch
            rc = lib.b200_paged_decode(q.data_ptr(), q.stride(0), k_pool.data_ptr(), v_pool.data_ptr(), table.data_ptr(),
                                       max_len_pages, seq_lens.data_ptr(), n, hq, self.kv_heads, D, float(scale), splits,
                                       out.data_ptr(), out.stride(0), _lib.ptr(scratch), _lib.stream_ptr())
            _lib.check_rc(rc, "paged_decode")
            ops._count(2 if splits > 1 else 1)
            return out
        return self._decode_reference(k_pool, v_pool, q, hq, table, seq_lens, scale)

    def _decode_reference(self, k_pool, v_pool, q, hq, table, seq_lens, scale):
        n, D, hkv = q.shape[0], self.head_dim, self.kv_heads
        out = torch.empty(n, hq * D, dtype=q.dtype, device=q.device)
        for i in range(n):
            L = int(seq_lens[i])
            pages = table[i, : (L + PAGE - 1) // PAGE].long()
            k = k_pool[pages].reshape(-1, hkv, D)[:L].transpose(0, 1).unsqueeze(0)   # [1,hkv,L,D]
            v = v_pool[pages].reshape(-1, hkv, D)[:L].transpose(0, 1).unsqueeze(0)
            qi = q[i].view(1, hq, 1, D)
            o = attn_ops.attention_reference(qi, k, v, causal=False, scale=scale)
            out[i] = o.reshape(-1)
        return out


class PagedKVAdaptor:
    """Connects fused Llama layers to a :class:`PagedKVCache`; the serving engine sets the batch context per step."""

    def __init__(self, cache: PagedKVCache):
        self.cache = cache
        self.mode = "prefill"
        self.table: Optional[torch.Tensor] = None       # int32 [n, blocks]: block-table rows of this step's sequences
        self.seq_idx: Optional[torch.Tensor] = None     # int32 [tokens]: row of ``table`` each token belongs to
        self.seq_lens: Optional[torch.Tensor] = None    # int32 [n], lengths including the new token (decode)

    def attend(self, layer, qkv: torch.Tensor, B: int, S: int, pos: torch.Tensor) -> torch.Tensor:
        hq, hkv, D = layer.hq, layer.hkv, layer.head_dim
        c = self.cache
        c.write(layer.layer_idx, qkv, hq, self.table, self.seq_idx, pos)
        if self.mode == "prefill":
            return attn_ops.causal_attention_packed(qkv, B, S, hq, hkv, D)
        return c.decode_attention(layer.layer_idx, qkv[:, : hq * D], hq, self.table, self.seq_lens)
