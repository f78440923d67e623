"""Block-selected ("sparse") decode attention for long contexts: a predictor scores the KV blocks of every sequence
against the current query and attention runs over a bounded number of blocks per sequence instead of all of them.

Per attention layer the selector keeps, for every physical KV block, the sum of its (rotated, dequantised) keys per KV
head and the number of tokens in it, recomputed from the cache for the blocks a step wrote to.  At a decode step a
block's score is ``max over kv heads of (mean query of the head's group) . (mean key of the block)``; the first
``sink`` blocks and the last ``recent`` blocks (the partly filled one included) are always kept, the rest of the
budget goes to the best-scoring blocks in between.  The result is a COMPACTED block table in position order plus the
matching sequence lengths, so the ordinary paged decode kernels run unchanged on fewer blocks: keys are already rotated
when they are cached, so attention over a subset needs no position fix-up, and the partly filled block stays last.
Everything is batched tensor work on the device with no host synchronisation, so a decode step stays capturable.

Sequences whose block count is within the budget are left exactly as they are (bit-identical attention).

This is the selection half of a tiered long-context KV store: blocks that are never selected do not have to be resident
on the device.  The streaming half (fetching selected blocks from the host / file tiers into scratch blocks before the
attention call) is not wired to it.

Reference parity: ``crates/spark-storage/src/predictor.rs`` (block scoring against a query projection),
``crates/spark-storage/src/high_speed_swap.rs`` (predictor + eviction + tiled attention orchestration),
``kernels/gb10/common/dsa_indexer.cu`` (pooled-key top-k selection).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch


class BlockSelector:
    def __init__(self, num_blocks: int, block_size: int, budget_blocks: int, sink: int = 1, recent: int = 2):
        assert budget_blocks >= sink + recent + 1, "budget must leave room for at least one selected block"
        self.num_blocks, self.bs = int(num_blocks), int(block_size)
        self.budget, self.sink, self.recent = int(budget_blocks), int(sink), int(recent)
        self.key_sum: Dict[int, torch.Tensor] = {}        # layer -> [num_blocks, Hkv, D] fp32
        self.count: Dict[int, torch.Tensor] = {}          # layer -> [num_blocks] fp32
        self.selected_steps = 0

    # ------------------------------------------------------------------ summaries
    def _buffers(self, layer: int, k_cache: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if layer not in self.key_sum:
            nb, _, hkv, d = k_cache.shape
            self.key_sum[layer] = torch.zeros(nb, hkv, d, dtype=torch.float32, device=k_cache.device)
            self.count[layer] = torch.zeros(nb, dtype=torch.float32, device=k_cache.device)
        return self.key_sum[layer], self.count[layer]

    @torch.no_grad()
    def on_write(self, layer: int, k_cache: torch.Tensor, batch, k_scale: float = 1.0) -> None:
        """Refresh the summaries of the blocks this step wrote to, from the cache contents (call after the KV write)."""
        ks, cnt = self._buffers(layer, k_cache)
        bs = self.bs
        if batch.num_decodes == batch.num_seqs:
            last = (batch.seq_lens.long() - 1)
            ids = batch.block_tables.long().gather(1, (last // bs)[:, None])[:, 0]
            n_valid = (last % bs + 1).float()
            self._refresh(ks, cnt, k_cache, ids, n_valid, k_scale)
            return
        # chunks: the host knows which table columns every chunk touched
        for b, (sl, ql) in enumerate(zip(batch.seq_lens_host, batch.query_lens_host)):
            lo, hi = (sl - ql) // bs, (sl - 1) // bs
            ids = batch.block_tables[b, lo:hi + 1].long()
            n_valid = torch.full((hi - lo + 1,), float(bs), device=ids.device)
            n_valid[-1] = float((sl - 1) % bs + 1)
            self._refresh(ks, cnt, k_cache, ids, n_valid, k_scale)

    def _refresh(self, ks, cnt, k_cache, ids, n_valid, k_scale) -> None:
        raw = k_cache.view(torch.uint8) if k_cache.element_size() == 1 else k_cache   # 8-bit floats are gathered as bytes
        kk = raw[ids]
        kk = (kk.view(k_cache.dtype) if k_cache.element_size() == 1 else kk).float()  # [n, bs, Hkv, D], logical order
        live = (torch.arange(self.bs, device=ids.device)[None, :] < n_valid[:, None]).float()
        ks[ids] = (kk * live[:, :, None, None]).sum(1) * k_scale
        cnt[ids] = n_valid

    # ------------------------------------------------------------------ selection
    @torch.no_grad()
    def select(self, layer: int, q: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
               ) -> Tuple[torch.Tensor, torch.Tensor]:
        """``q [B, Hq, D]`` (one decode row per sequence) -> (compacted tables ``[B, budget]``, sequence lengths)."""
        ks, cnt = self.key_sum[layer], self.count[layer]
        B, Hq, D = q.shape
        hkv = ks.shape[1]
        bs, W = self.bs, self.budget
        maxb = block_tables.shape[1]
        L = seq_lens.long()
        n_blk = (L + bs - 1) // bs
        if maxb <= W:
            return block_tables, seq_lens
        tab = block_tables.long()
        qg = q.float().view(B, hkv, Hq // hkv, D).mean(2)                                   # [B, Hkv, D]
        mean_k = ks[tab] / cnt[tab].clamp_min(1.0)[..., None, None]                          # [B, maxb, Hkv, D]
        score = torch.einsum("bhd,bjhd->bjh", qg, mean_k).amax(-1)                           # [B, maxb]
        j = torch.arange(maxb, device=q.device)[None, :]
        valid = j < n_blk[:, None]
        forced = (j < self.sink) | (j >= (n_blk - self.recent)[:, None])
        score = torch.where(forced, torch.full_like(score, float("inf")), score)
        score = torch.where(valid, score, torch.full_like(score, float("-inf")))
        # ties at +inf / -inf resolve by index through the stable sort below: keep position order inside every class
        pick = torch.topk(score, W, dim=1, sorted=False).indices
        pick = torch.sort(pick, dim=1).values                                                # position order, last block last
        # sequences within the budget picked some invalid columns: they sort to the end and are never read
        new_tab = tab.gather(1, pick).to(block_tables.dtype)
        tail = L - (n_blk - 1) * bs                                                          # tokens in the last block
        new_len = torch.where(n_blk > W, (W - 1) * bs + tail, L).to(seq_lens.dtype)
        self.selected_steps += 1
        return new_tab, new_len


def attend_selected(ops_paged_attention, selector: Optional[BlockSelector], layer: int, q, k_cache, v_cache, batch, scale,
                    k_scale, v_scale, window):
    """Decode attention through ``selector`` when it applies to this step, plain paged attention otherwise."""
    if selector is None or batch.num_decodes != batch.num_seqs or batch.num_seqs == 0 or window:
        return ops_paged_attention(q, k_cache, v_cache, batch, scale, k_scale, v_scale, window)
    tab, lens = selector.select(layer, q, batch.block_tables, batch.seq_lens)
    if tab is batch.block_tables:
        return ops_paged_attention(q, k_cache, v_cache, batch, scale, k_scale, v_scale, window)
    sub = dataclasses.replace(batch, block_tables=tab, seq_lens=lens,
                              max_seq_len=min(batch.max_seq_len, selector.budget * selector.bs))
    for name in ("_attn_tiles", "_mrope"):
        if hasattr(sub, name):
            delattr(sub, name)
    return ops_paged_attention(q, k_cache, v_cache, sub, scale, k_scale, v_scale, window)
