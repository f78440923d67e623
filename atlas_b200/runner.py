"""ModelRunner: turns a scheduler plan into device tensors, runs the model, returns logits rows.

On a GPU the runner keeps pinned host staging buffers (one H2D copy per metadata tensor per step) and
replays a captured CUDA graph for pure-decode batches, keyed by the padded batch size, with the
batch tensors living at fixed addresses (reference: graph cache keyed ``(padded_n, family)`` in
``crates/spark-model/src/model/trait_impl/decode_a2.rs:408-620``).  On CPU it simply runs the eager
model.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .config import EngineConfig
from .models import CacheStore, DecoderLM, ForwardBatch
from .sched import SchedulerOutput

_GRAPH_BATCH_SIZES = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def _pad_batch(n: int) -> int:
    for b in _GRAPH_BATCH_SIZES:
        if n <= b:
            return b
    return n


class ModelRunner:
    def __init__(self, model: DecoderLM, cache: CacheStore, cfg: EngineConfig):
        self.model, self.cache, self.cfg = model, cache, cfg
        self.device = model.device
        self.bs = cfg.block_size
        self.on_gpu = self.device.type == "cuda"
        self.max_blocks_per_seq = (cfg.max_seq_len + self.bs - 1) // self.bs
        self.graphs: Dict[int, "_DecodeGraph"] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_replays = 0
        self._pin: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ batch assembly
    def _stage(self, name: str, data: List[int], dtype: torch.dtype) -> torch.Tensor:
        """Host list -> device tensor through a reusable pinned buffer (one async H2D copy)."""
        n = len(data)
        if not self.on_gpu:
            return torch.tensor(data, dtype=dtype)
        buf = self._pin.get(name)
        if buf is None or buf.numel() < n or buf.dtype != dtype:
            cap = max(1024, 1 << (max(n, 1) - 1).bit_length())
            buf = torch.empty(cap, dtype=dtype, pin_memory=True)
            self._pin[name] = buf
        host = buf[:n]
        host.copy_(torch.tensor(data, dtype=dtype))
        self.h2d_bytes += host.numel() * host.element_size()
        return host.to(self.device, non_blocking=True)

    def build_batch(self, out: SchedulerOutput, snapshot_base: int = 0) -> ForwardBatch:
        bs = self.bs
        ids: List[int] = []
        pos: List[int] = []
        slots: List[int] = []
        qsl = [0]
        sl: List[int] = []
        qlens: List[int] = []
        tables: List[List[int]] = []
        state_slots: List[int] = []
        has_state: List[bool] = []
        num_dec = 0
        spec_verify = False
        for it in out.items:
            seq = it.seq
            if it.verify_drafts:
                toks = [seq.all_tokens[it.start]] + list(seq.drafts[:it.verify_drafts])
                spec_verify = True
            else:
                toks = seq.all_tokens[it.start:it.start + it.num_tokens]
            if it.is_decode:
                num_dec += 1
            blocks = seq.blocks
            for j, t in enumerate(toks):
                p = it.start + j
                ids.append(t)
                pos.append(p)
                slots.append(blocks[p // bs] * bs + p % bs)
            qsl.append(qsl[-1] + len(toks))
            sl.append(it.start + len(toks))
            qlens.append(len(toks))
            tables.append(blocks)
            state_slots.append(seq.state_slot if seq.state_slot is not None else 0)
            has_state.append(seq.has_state)
        B = len(out.items)
        maxb = max(len(t) for t in tables)
        flat_tables: List[int] = []
        for t in tables:
            flat_tables.extend(t)
            flat_tables.extend([0] * (maxb - len(t)))
        fb = ForwardBatch(
            input_ids=self._stage("ids", ids, torch.int64),
            positions=self._stage("pos", pos, torch.int32),
            slot_mapping=self._stage("slots", slots, torch.int32),
            block_tables=self._stage("tables", flat_tables, torch.int32).view(B, maxb),
            seq_lens=self._stage("sl", sl, torch.int32),
            query_start_loc=self._stage("qsl", qsl, torch.int32),
            num_decodes=num_dec, max_query_len=max(qlens), max_seq_len=max(sl),
            seq_lens_host=sl, query_lens_host=qlens, spec_verify=spec_verify,
        )
        if self.model.gdn_layers():
            fb.state_slots = self._stage("state_slots", state_slots, torch.int32)
            fb.state_slots_host, fb.has_state_host = state_slots, has_state
        for item_idx, rows, slot in out.snapshot_requests:
            fb.snapshot_plan.setdefault(item_idx, []).append((rows, snapshot_base + slot))
        return fb

    # ------------------------------------------------------------------ execution
    def _can_graph(self, batch: ForwardBatch) -> bool:
        return (self.on_gpu and self.cfg.use_cuda_graphs and batch.num_seqs > 0
                and batch.num_decodes == batch.num_seqs and not batch.spec_verify
                and getattr(self.model, "graph_safe", True) and not self.model.gdn_layers())

    def forward(self, batch: ForwardBatch) -> torch.Tensor:
        if self._can_graph(batch):
            return self._forward_graph(batch)
        return self.model.forward(batch, self.cache)

    def kernels_per_graph(self) -> int:
        """Kernel launches inside one captured decode step (what one replay stands for)."""
        ks = [g.num_kernels for g in self.graphs.values() if g.num_kernels]
        return int(sum(ks) / len(ks)) if ks else 0

    def logits(self, hidden: torch.Tensor, rows: List[int]) -> torch.Tensor:
        if len(rows) == hidden.shape[0] and rows == list(range(len(rows))):
            return self.model.compute_logits(hidden)
        idx = self._stage("rows", rows, torch.int64)
        return self.model.compute_logits(hidden, idx)

    def copy_state(self, src_slot: int, dst_slot: int) -> None:
        for st in self.cache.states.values():
            st["conv"][dst_slot].copy_(st["conv"][src_slot])
            st["h"][dst_slot].copy_(st["h"][src_slot])

    # ------------------------------------------------------------------ CUDA graphs (decode)
    def _forward_graph(self, batch: ForwardBatch) -> torch.Tensor:
        B = batch.num_seqs
        P = _pad_batch(B)
        g = self.graphs.get(P)
        if g is None:
            g = _DecodeGraph(self, P)
            self.graphs[P] = g
        return g.run(batch)


class _DecodeGraph:
    """One captured decode step for a padded batch size; inputs are copied into fixed buffers."""

    def __init__(self, runner: ModelRunner, padded: int):
        self.r, self.P = runner, padded
        dev = runner.device
        mb = runner.max_blocks_per_seq
        self.ids = torch.zeros(padded, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(padded, dtype=torch.int32, device=dev)
        self.slots = torch.full((padded,), -1, dtype=torch.int32, device=dev)
        self.tables = torch.zeros(padded, mb, dtype=torch.int32, device=dev)
        self.seq_lens = torch.ones(padded, dtype=torch.int32, device=dev)
        self.qsl = torch.arange(padded + 1, dtype=torch.int32, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.num_kernels = 0

    def _batch(self, max_seq_len: int) -> ForwardBatch:
        return ForwardBatch(input_ids=self.ids, positions=self.pos, slot_mapping=self.slots, block_tables=self.tables,
                            seq_lens=self.seq_lens, query_start_loc=self.qsl, num_decodes=self.P, max_query_len=1,
                            max_seq_len=max_seq_len, seq_lens_host=[1] * self.P, query_lens_host=[1] * self.P)

    def _load(self, b: ForwardBatch) -> None:
        n = b.num_seqs
        self.ids[:n].copy_(b.input_ids, non_blocking=True)
        self.pos[:n].copy_(b.positions, non_blocking=True)
        self.slots[:n].copy_(b.slot_mapping, non_blocking=True)
        self.seq_lens[:n].copy_(b.seq_lens, non_blocking=True)
        self.tables[:n, :b.block_tables.shape[1]].copy_(b.block_tables, non_blocking=True)
        if n < self.P:
            self.slots[n:].fill_(-1)
            self.seq_lens[n:].fill_(1)
            self.ids[n:].zero_()
            self.pos[n:].zero_()

    def run(self, b: ForwardBatch) -> torch.Tensor:
        self._load(b)
        r = self.r
        if self.graph is None:
            # the graph must be valid for any later sequence length: kernels read lengths from device memory
            fb = self._batch(r.cfg.max_seq_len)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    r.model.forward(fb, r.cache)
            torch.cuda.current_stream().wait_stream(s)
            self.graph = torch.cuda.CUDAGraph()
            from .ops import cuda as K
            n0 = K.launch_count
            with torch.cuda.graph(self.graph):
                self.out = r.model.forward(fb, r.cache)
            self.num_kernels = K.launch_count - n0
            self._load(b)
        self.graph.replay()
        r.graph_replays += 1
        return self.out[:b.num_seqs]
