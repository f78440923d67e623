"""ModelRunner: turns a scheduler plan into device tensors, runs the model, returns logits rows.

On a GPU the runner keeps pinned host staging buffers (one H2D copy per metadata tensor per step) and
replays a captured CUDA graph for pure-decode batches, keyed by the padded batch size, with the
batch tensors living at fixed addresses (reference: graph cache keyed ``(padded_n, family)`` in
``crates/spark-model/src/model/trait_impl/decode_a2.rs:408-620``).  On CPU it simply runs the eager
model.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
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
        if self.on_gpu:
            self._reserve_attention_scratch()

    def graph_batch_sizes(self) -> List[int]:
        """Every batch size a decode step can be padded to under this configuration."""
        top = max(self.cfg.max_batch_size, self.cfg.max_num_seqs)
        sizes = [b for b in _GRAPH_BATCH_SIZES if b <= top]
        sizes.append(_pad_batch(top))
        return sorted(set(sizes + list(range(1, min(top, 8) + 1))))

    def _reserve_attention_scratch(self) -> None:
        """Size the split-K decode attention scratch for the largest case any later step can ask for, so that the
        buffers captured into CUDA graphs are never replaced."""
        from .ops import cuda as K
        mixers = [l.mixer for l in self.model.layers if l.kind == "attention"]
        if getattr(self.model, "mtp", None) is not None and getattr(self.model.mtp, "layer", None) is not None:
            mixers.append(self.model.mtp.layer.mixer)
        if not mixers:
            return
        d = K._dev(torch.empty(1, device=self.device))
        sms = K._num_sms[d]
        top = max(self.graph_batch_sizes())            # eager mixed steps can carry any number of decode rows up to this
        sizes = list(range(1, top + 1))
        po = pml = 0
        for m in mixers:
            a, b = K.attention_scratch_bytes(sizes, m.hq, m.hkv, m.d, self.cfg.max_seq_len, sms)
            po, pml = max(po, a), max(pml, b)
        if po:
            K.reserve_scratch("attn_part_o", po, self.device)
            K.reserve_scratch("attn_part_ml", pml, self.device)

    # ------------------------------------------------------------------ batch assembly
    def _stage(self, name: str, data, dtype: torch.dtype) -> torch.Tensor:
        """Host list / numpy array -> device tensor through a reusable pinned buffer (one async H2D copy)."""
        src = torch.from_numpy(data) if isinstance(data, np.ndarray) else torch.tensor(data, dtype=dtype)
        if src.dtype != dtype:
            src = src.to(dtype)
        n = src.numel()
        if not self.on_gpu:
            return src.reshape(-1)
        buf = self._pin.get(name)
        if buf is None or buf.numel() < n or buf.dtype != dtype:
            cap = max(1024, 1 << (max(n, 1) - 1).bit_length())
            buf = torch.empty(cap, dtype=dtype, pin_memory=True)
            self._pin[name] = buf
        host = buf[:n]
        host.copy_(src.reshape(-1))
        self.h2d_bytes += n * host.element_size()
        return host.to(self.device, non_blocking=True)

    @staticmethod
    def _blocks_np(seq) -> np.ndarray:
        """Block table of a sequence as a cached int32 array (rebuilt only when the list changed length)."""
        cached = getattr(seq, "_blocks_cache", None)
        blocks = seq.blocks
        if cached is None or cached[0] != len(blocks) or cached[2] is not blocks:
            cached = (len(blocks), np.asarray(blocks, dtype=np.int32), blocks)
            seq._blocks_cache = cached
        elif len(blocks) and cached[1][-1] != blocks[-1]:
            cached = (len(blocks), np.asarray(blocks, dtype=np.int32), blocks)
            seq._blocks_cache = cached
        return cached[1]

    def build_batch(self, out: SchedulerOutput, snapshot_base: int = 0) -> ForwardBatch:
        bs = self.bs
        items = out.items
        B = len(items)
        tabs = [self._blocks_np(it.seq) for it in items]
        maxb = max(t.shape[0] for t in tabs)
        table = np.zeros((B, maxb), dtype=np.int32)
        for i, t in enumerate(tabs):
            table[i, :t.shape[0]] = t
        state_slots = [it.seq.state_slot if it.seq.state_slot is not None else 0 for it in items]
        has_state = [it.seq.has_state for it in items]
        spec_verify = False
        any_mm = any(getattr(it.seq, "mm", None) is not None for it in items)
        if not any_mm and all(it.num_tokens == 1 and not it.verify_drafts for it in items):
            # every row is one token of one sequence (decode, or a one-token chunk): vectorised
            starts = np.fromiter((it.start for it in items), dtype=np.int64, count=B)
            ids = np.fromiter((it.seq.token_at(it.start) for it in items), dtype=np.int64, count=B)
            pos = starts.astype(np.int32)
            blk = table[np.arange(B), starts // bs]
            slots = (blk.astype(np.int64) * bs + starts % bs).astype(np.int32)
            qsl = np.arange(B + 1, dtype=np.int32)
            sl_np = (starts + 1).astype(np.int32)
            sl = sl_np.tolist()
            qlens = [1] * B
            num_dec = sum(1 for it in items if it.is_decode)
        else:
            ids_l: List[int] = []
            pos_l: List[int] = []
            slots_l: List[int] = []
            qsl_l = [0]
            sl = []
            qlens = []
            num_dec = 0
            for i, it in enumerate(items):
                seq = it.seq
                if it.verify_drafts:
                    toks = [seq.token_at(it.start)] + list(seq.drafts[:it.verify_drafts])
                    spec_verify = True
                else:
                    toks = seq.tokens_range(it.start, it.start + it.num_tokens)
                if it.is_decode:
                    num_dec += 1
                n = len(toks)
                p = np.arange(it.start, it.start + n, dtype=np.int64)
                ids_l.extend(toks)
                pos_l.append(p)
                slots_l.append(tabs[i][p // bs].astype(np.int64) * bs + p % bs)
                qsl_l.append(qsl_l[-1] + n)
                sl.append(it.start + n)
                qlens.append(n)
            ids = np.asarray(ids_l, dtype=np.int64)
            pos = np.concatenate(pos_l).astype(np.int32)
            slots = np.concatenate(slots_l).astype(np.int32)
            qsl = np.asarray(qsl_l, dtype=np.int32)
            sl_np = np.asarray(sl, dtype=np.int32)
        fb = ForwardBatch(
            input_ids=self._stage("ids", ids, torch.int64),
            positions=self._stage("pos", pos, torch.int32),
            slot_mapping=self._stage("slots", slots, torch.int32),
            block_tables=self._stage("tables", table, torch.int32).view(B, maxb),
            seq_lens=self._stage("sl", sl_np, torch.int32),
            query_start_loc=self._stage("qsl", qsl, torch.int32),
            num_decodes=num_dec, max_query_len=max(qlens), max_seq_len=max(sl),
            seq_lens_host=sl, query_lens_host=qlens, spec_verify=spec_verify,
        )
        if any_mm:
            self._add_multimodal(fb, items, ids, qlens)
        if any(it.seq.adapter_slot for it in items):
            fb.adapter_rows = self._stage("adapter_rows", np.repeat(np.asarray([it.seq.adapter_slot for it in items], dtype=np.int64),
                                                                    np.asarray(qlens)), torch.int64)
        if self.model.gdn_layers():
            fb.state_slots = self._stage("state_slots", state_slots, torch.int32)
            fb.state_slots_host, fb.has_state_host = state_slots, has_state
        for item_idx, rows, slot in out.snapshot_requests:
            fb.snapshot_plan.setdefault(item_idx, []).append((rows, snapshot_base + slot))
        return fb

    def _add_multimodal(self, fb: ForwardBatch, items, ids: np.ndarray, qlens: List[int]) -> None:
        """Three-stream rotary positions for every row and, where a chunk covers image placeholders, input embeddings
        with those rows replaced by the vision tower's output."""
        p3 = []
        rows, src_seq, src_row = [], [], []
        r0 = 0
        for it, n in zip(items, qlens):
            mm = getattr(it.seq, "mm", None)
            if mm is None:
                p3.append(np.broadcast_to(np.arange(it.start, it.start + n, dtype=np.int64), (3, n)))
            else:
                p3.append(mm.positions(it.start, it.start + n))
                hi = min(it.start + n, mm.index_of.shape[0])
                if hi > it.start:
                    idx = mm.index_of[it.start:hi]
                    for j in np.nonzero(idx >= 0)[0]:
                        rows.append(r0 + int(j))
                        src_seq.append(it.seq)
                        src_row.append(int(idx[j]))
            r0 += n
        fb.positions3 = self._stage("pos3", np.ascontiguousarray(np.concatenate(p3, 1)), torch.int64).view(3, -1)
        if rows:
            emb = self.model.embed_tokens(fb.input_ids).clone()
            by_seq: dict = {}
            for r, s, j in zip(rows, src_seq, src_row):
                by_seq.setdefault(id(s), (s, [], []))
                by_seq[id(s)][1].append(r)
                by_seq[id(s)][2].append(j)
            for s, rr, jj in by_seq.values():
                src = s.mm.embeds.to(device=emb.device, dtype=emb.dtype)
                emb[torch.tensor(rr, device=emb.device)] = src[torch.tensor(jj, device=emb.device)]
            fb.inputs_embeds = emb

    # ------------------------------------------------------------------ execution
    def _can_graph(self, batch: ForwardBatch) -> bool:
        return (self.on_gpu and self.cfg.use_cuda_graphs and batch.num_seqs > 0
                and batch.num_decodes == batch.num_seqs and not batch.spec_verify and batch.adapter_rows is None
                and batch.positions3 is None
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

    def greedy_tokens(self, hidden: torch.Tensor, rows: List[int]) -> torch.Tensor:
        if len(rows) == hidden.shape[0] and rows == list(range(len(rows))):
            return self.model.greedy_tokens(hidden)
        return self.model.greedy_tokens(hidden, self._stage("rows", rows, torch.int64))

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
            K.freeze_scratch()
            n0 = K.launch_count
            with torch.cuda.graph(self.graph):
                self.out = r.model.forward(fb, r.cache)
            self.num_kernels = K.launch_count - n0
            self._load(b)
        self.graph.replay()
        r.graph_replays += 1
        return self.out[:b.num_seqs]
