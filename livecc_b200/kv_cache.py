"""Paged KV cache: the object that lives in `state['past_key_values']` between `generate()` calls.

Replaces transformers' DynamicCache/DynamicLayer (cache_utils.py:88-163), which re-concatenates the
whole K and V of every layer on every token (`torch.cat`, :119-120). Here a stream owns a list of
64-token pages inside one pool per engine; appending a token writes 2*layers*kv_heads*128 bf16 and
never moves old data. The per-stream rope_delta (kept on the *model* by the reference,
mq2vl.py:923) lives here, so any number of streams can interleave on one engine.

Pool layout (HBM): K and V pools are bf16 [layers, num_pages, kv_heads, 64, 128]; a layer's pool is
contiguous so a (page, head) tile is one 16 KB run — coalesced for the decode kernel and TMA-shaped.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ._cabi import PAGE_SIZE, SC_COUNT, StreamState


class PageAllocator:
    """Free list of fixed-size pages; storage is the subclass's (`_resize_storage` re-creates it for a new page count and
    copies the old pages over). Grows by doubling (rare)."""

    def __init__(self, device, initial_pages: int):
        self.device = device
        self.num_pages = 0
        self.free: List[int] = []
        self.generation = 0  # bumped whenever the pool storage moves (invalidates captured graphs)
        self._grow(initial_pages)

    def _resize_storage(self, new_total: int):
        raise NotImplementedError

    def _grow(self, new_total: int):
        self._resize_storage(new_total)
        self.free.extend(range(self.num_pages, new_total))
        self.num_pages = new_total
        self.generation += 1

    def alloc(self, n: int) -> List[int]:
        while len(self.free) < n:
            self._grow(max(self.num_pages * 2, self.num_pages + n))
        out = self.free[:n]
        del self.free[:n]
        return out

    def release(self, pages: List[int]):
        self.free.extend(pages)


class PagePool(PageAllocator):
    """Fixed-size pages shared by all streams of one engine (every layer has the same K/V geometry, head size 128)."""

    def __init__(self, layers: int, kv_heads: int, device, initial_pages: int = 160):
        self.layers, self.kv_heads = layers, kv_heads
        self.k = self.v = None
        self._free_buffers: List["StreamBuffers"] = []
        super().__init__(device, initial_pages)

    def _resize_storage(self, new_total: int):
        shape = (self.layers, new_total, self.kv_heads, PAGE_SIZE, 128)
        k = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        v = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        if self.k is not None:
            k[:, : self.num_pages].copy_(self.k)
            v[:, : self.num_pages].copy_(self.v)
        self.k, self.v = k, v

    @property
    def layer_stride(self) -> int:
        return self.num_pages * self.kv_heads * PAGE_SIZE * 128

    # Per-stream device buffers (page table, scalars, id buffer) are recycled through the pool so that their
    # addresses — which are baked into captured decode graphs — stay stable from one stream to the next.
    def acquire_buffers(self) -> "StreamBuffers":
        return self._free_buffers.pop() if self._free_buffers else StreamBuffers(self.device)

    def release_buffers(self, b: "StreamBuffers"):
        self._free_buffers.append(b)

    def bytes_per_token(self) -> int:
        return 2 * self.layers * self.kv_heads * 128 * 2


class StreamBuffers:
    def __init__(self, device):
        self.page_table = torch.zeros(512, dtype=torch.int32, device=device)   # 32k tokens before the first growth
        self.scalars = torch.zeros(SC_COUNT, dtype=torch.int32, device=device)
        self.seq_buf = torch.zeros(32768, dtype=torch.int64, device=device)
        self.generation = 0


class PagedKVCache:
    """One stream's cache: page list, sequence length, rope_delta, device scalars and the id buffer."""

    def __init__(self, pool: PagePool):
        self.pool = pool
        self.pages: List[int] = []
        self.seq_len = 0                       # tokens whose K/V are in the cache
        self.rope_delta: Optional[int] = None  # turn-0 value, never updated (mq2vl.py:1207,1518)
        self._buf = pool.acquire_buffers()
        self._pages_uploaded = 0

    # the buffers live in a recyclable slot; expose them under their old names
    @property
    def page_table(self):
        return self._buf.page_table

    @property
    def scalars(self):
        return self._buf.scalars

    @property
    def seq_buf(self):
        return self._buf.seq_buf

    @property
    def buffers_generation(self):
        return self._buf.generation

    # -- HF Cache surface used by callers (gen/utils.py:3748) -----------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.seq_len

    def __len__(self):
        return self.pool.layers

    # -- capacity --------------------------------------------------------------------------------
    def ensure_tokens(self, n_tokens: int):
        need = (n_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        if need > len(self.pages):
            self.pages.extend(self.pool.alloc(need - len(self.pages)))
        if need > self.page_table.numel():
            self._buf.page_table = torch.zeros(max(need, 2 * self.page_table.numel()), dtype=torch.int32,
                                               device=self.pool.device)
            self._pages_uploaded = 0
            self._buf.generation += 1
        if self._pages_uploaded < len(self.pages):
            host = torch.tensor(self.pages[self._pages_uploaded:], dtype=torch.int32)
            self.page_table[self._pages_uploaded:len(self.pages)].copy_(host, non_blocking=False)
            self._pages_uploaded = len(self.pages)

    def ensure_seq_capacity(self, n_ids: int):
        if n_ids > self.seq_buf.numel():
            self._buf.seq_buf = torch.zeros(max(n_ids, 2 * self.seq_buf.numel()), dtype=torch.int64,
                                            device=self.pool.device)
            self._buf.generation += 1

    def stream_state(self) -> StreamState:
        p = self.pool
        return StreamState(p.k.data_ptr(), p.v.data_ptr(), p.layer_stride, self.page_table.data_ptr(),
                           self.scalars.data_ptr(), self.seq_buf.data_ptr())

    def graph_key(self):
        return (self.pool.generation, self.buffers_generation, self.page_table.data_ptr(), self.scalars.data_ptr(),
                self.seq_buf.data_ptr())

    def release(self):
        """Return the pages to the pool (end of stream)."""
        if self.pages:
            self.pool.release(self.pages)
            self.pages = []
        if self._buf is not None:
            self.pool.release_buffers(self._buf)
            self._buf = None
        self.seq_len = 0
        self.rope_delta = None
        self._pages_uploaded = 0

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    # -- debugging / parity ------------------------------------------------------------------------
    def gather(self, layer: int):
        """Logical (K, V) of one layer as [kv_heads, seq_len, 128] tensors (test helper)."""
        n = (self.seq_len + PAGE_SIZE - 1) // PAGE_SIZE
        idx = torch.tensor(self.pages[:n], dtype=torch.long, device=self.pool.device)
        k = self.pool.k[layer][idx].permute(1, 0, 2, 3).reshape(self.pool.kv_heads, -1, 128)[:, : self.seq_len]
        v = self.pool.v[layer][idx].permute(1, 0, 2, 3).reshape(self.pool.kv_heads, -1, 128)[:, : self.seq_len]
        return k, v


# ------------------------------------------------------------------------------------------------
# Hybrid sequence models: pages for the attention layers + fp32 state slots for the recurrent layers
# ------------------------------------------------------------------------------------------------
class SeqStatePool(PageAllocator):
    """Memory of every live sequence of one hybrid-model engine.

    * Attention layers: K pages [num_pages, kv_heads, PAGE_SIZE, dim] and V pages [num_pages, kv_heads, PAGE_SIZE, vdim]
      per layer (layers may differ in geometry; page ids are shared by all layers). A chunk-local layer never looks
      behind the start of the current chunk, so a sequence gives pages back as soon as every attention layer has left them.
      vdim = 0: the layer keeps K pages only (a latent cache, whose values are channels of the key rows); a layer that
      reads another layer's cache has no entry here.
    * Recurrent layers: one fp32 slot per sequence and layer (`state_floats[i]` elements, 0 for none), zeroed when a
      sequence takes it.
    attn_layers: {layer index: (kv_heads, dim, vdim, chunk[, window])}; state_floats: per layer. A layer with a sliding
    window of w positions never looks more than w - 1 positions behind the newest token."""

    def __init__(self, attn_layers: dict, state_floats: List[int], dtype, device, initial_pages: int = 32, initial_slots: int = 2):
        self.attn_layers = dict(attn_layers)
        self.state_floats = list(state_floats)
        self.dtype = dtype
        self.k = {i: None for i in self.attn_layers}
        self.v = {i: None for i in self.attn_layers}
        self.num_slots = 0
        self.free_slots: List[int] = []
        self.state: List[Optional[torch.Tensor]] = [None] * len(self.state_floats)
        super().__init__(device, max(1, initial_pages) if self.attn_layers else 0)
        self.device = device
        self._grow_slots(max(1, initial_slots))

    # pages ------------------------------------------------------------------------------------
    def _resize_storage(self, new_total: int):
        for i, (g, d, dv, *_mask) in self.attn_layers.items():
            k = torch.zeros((new_total, g, PAGE_SIZE, d), dtype=self.dtype, device=self.device)
            v = torch.zeros((new_total, g, PAGE_SIZE, dv), dtype=self.dtype, device=self.device) if dv else None
            if self.k[i] is not None:
                k[: self.num_pages].copy_(self.k[i])
                if v is not None:
                    v[: self.num_pages].copy_(self.v[i])
            self.k[i], self.v[i] = k, v

    def keep_from(self, seq_len: int) -> int:
        """First position any attention layer can still read once `seq_len` tokens are cached."""
        if not self.attn_layers:
            return seq_len
        lo = seq_len
        for (_g, _d, _dv, chunk, *rest) in self.attn_layers.values():
            first = (seq_len // chunk) * chunk if chunk > 0 else 0
            if rest and rest[0] > 0:       # the next token sits at position seq_len and sees seq_len - window + 1 onwards
                first = max(first, seq_len - rest[0] + 1)
            lo = min(lo, first)
        return lo

    # state slots ------------------------------------------------------------------------------
    def _grow_slots(self, new_total: int):
        for i, n in enumerate(self.state_floats):
            if n <= 0:
                continue
            t = torch.zeros((new_total, n), dtype=torch.float32, device=self.device)
            if self.state[i] is not None:
                t[: self.num_slots].copy_(self.state[i])
            self.state[i] = t
        self.free_slots.extend(range(self.num_slots, new_total))
        self.num_slots = new_total
        self.generation += 1

    def acquire_slot(self) -> int:
        if not self.free_slots:
            self._grow_slots(self.num_slots * 2)
        slot = self.free_slots.pop()      # the slot freed last is used first
        for t in self.state:
            if t is not None:
                t[slot].zero_()   # a sequence starts from the zero state, whoever used the slot before
        return slot

    def release_slot(self, slot: int):
        self.free_slots.append(slot)

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g * (d + dv) * es for (g, d, dv, *_m) in self.attn_layers.values())

    def state_bytes_per_sequence(self) -> int:
        return 4 * sum(self.state_floats)


class SeqCache:
    """One sequence of a hybrid model: its state slot, its pages, its length, and (for generation) the device scalars and
    id buffer that the token-selection kernel advances. The HF-cache surface (`get_seq_length`) matches PagedKVCache."""

    def __init__(self, pool: SeqStatePool):
        self.pool = pool
        self.slot: Optional[int] = pool.acquire_slot()
        self.pages: List[Optional[int]] = []   # logical page -> physical page, None once given back
        self.seq_len = 0
        self.page_table = torch.zeros(64, dtype=torch.int32, device=pool.device)
        self.scalars = torch.zeros(SC_COUNT, dtype=torch.int32, device=pool.device)
        self.seq_buf: Optional[torch.Tensor] = None
        self.table_generation = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.seq_len

    def ensure_tokens(self, n_tokens: int):
        """Pages for positions [keep_from(seq_len), n_tokens)."""
        if not self.pool.attn_layers:
            return
        need = (n_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        first_new = len(self.pages)
        if need > first_new:
            self.pages.extend(self.pool.alloc(need - first_new))
            if need > self.page_table.numel():
                t = torch.zeros(max(need, 2 * self.page_table.numel()), dtype=torch.int32, device=self.pool.device)
                t[: self.page_table.numel()].copy_(self.page_table)
                self.page_table = t
                self.table_generation += 1
            host = torch.tensor(self.pages[first_new:need], dtype=torch.int32)
            self.page_table[first_new:need].copy_(host)

    def ensure_seq_capacity(self, n_ids: int):
        if self.seq_buf is None or n_ids > self.seq_buf.numel():
            t = torch.zeros(max(n_ids, 1024, 2 * (self.seq_buf.numel() if self.seq_buf is not None else 0)),
                            dtype=torch.int64, device=self.pool.device)
            if self.seq_buf is not None:
                t[: self.seq_buf.numel()].copy_(self.seq_buf)
            self.seq_buf = t
            self.table_generation += 1

    def advance(self, n_new: int):
        """`n_new` more tokens are cached; pages every attention layer has left go back to the pool."""
        self.seq_len += n_new
        last_dead = self.pool.keep_from(self.seq_len) // PAGE_SIZE
        dead = [p for p in self.pages[:last_dead] if p is not None]
        if dead:
            self.pool.release(dead)
            for i in range(min(last_dead, len(self.pages))):
                self.pages[i] = None

    def live_pages(self) -> int:
        return sum(p is not None for p in self.pages)

    def release(self):
        if self.slot is not None:
            self.pool.release_slot(self.slot)
            self.slot = None
        live = [p for p in self.pages if p is not None]
        if live:
            self.pool.release(live)
        self.pages = []
        self.seq_len = 0

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass
