"""Per-step tensors handed to ``DecoderLM.forward`` (continuous batching, flattened over tokens)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class ForwardBatch:
    """One engine step.

    Sequences are ordered decodes first (one query row each) and then prefill / verify chunks.
    Sequence ``b`` owns query rows ``query_start_loc[b]:query_start_loc[b+1]``; after this step its
    cache holds ``seq_lens[b]`` tokens.  Reference counterpart: ``ForwardContext``
    (``crates/spark-model/src/layer.rs:287``) plus the paged metadata uploads of
    ``model/trait_impl/prefill_b/upload_meta.rs``.
    """
    input_ids: torch.Tensor            # [T] int64
    positions: torch.Tensor            # [T] int32
    slot_mapping: torch.Tensor         # [T] int32 (-1 = padding)
    block_tables: torch.Tensor         # [B, max_blocks] int32
    seq_lens: torch.Tensor             # [B] int32
    query_start_loc: torch.Tensor      # [B+1] int32
    num_decodes: int = 0
    max_query_len: int = 1
    max_seq_len: int = 0
    logits_indices: Optional[torch.Tensor] = None   # rows whose logits are needed
    # host mirrors (no device sync needed by python-side loops)
    seq_lens_host: List[int] = field(default_factory=list)
    query_lens_host: List[int] = field(default_factory=list)
    # hybrid (GDN) models: recurrent-state slot per sequence, and whether that slot holds a live state
    state_slots: Optional[torch.Tensor] = None      # [B] int32
    has_state_host: List[bool] = field(default_factory=list)
    state_slots_host: List[int] = field(default_factory=list)
    # speculative verify: do not commit recurrent state, keep per-row inputs for a later fold
    spec_verify: bool = False
    # recurrent-state snapshots to take mid-chunk: {sequence index: [(rows from chunk start, dest slot)]}
    snapshot_plan: Dict[int, List[Tuple[int, int]]] = field(default_factory=dict)
    # optional precomputed input embeddings (MTP head / multimodal rows)
    inputs_embeds: Optional[torch.Tensor] = None
    # multimodal: three rotary position streams (time, row, column) per row; None for text-only steps
    positions3: Optional[torch.Tensor] = None       # [3, T] int64
    # LoRA: adapter slot of every row (0 = base model); None when no row of the step uses an adapter
    adapter_rows: Optional[torch.Tensor] = None

    def rope_inputs(self, rope_cache: torch.Tensor, mrope_section):
        """(positions, rotary table) for the fused rope kernels: the model's table indexed by position for text-only
        steps, a step-local table with one row per token (``positions = arange``) when three position streams are set."""
        if self.positions3 is None:
            return self.positions, rope_cache
        hit = getattr(self, "_mrope", None)
        if hit is None or hit[0] is not rope_cache:
            from .vision import mrope_table
            table = mrope_table(rope_cache, self.positions3, mrope_section or [11, 11, 10])
            hit = self._mrope = (rope_cache, torch.arange(table.shape[0], dtype=torch.int32, device=table.device), table)
        return hit[1], hit[2]

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0]) if self.input_ids is not None else int(self.inputs_embeds.shape[0])

    @property
    def num_seqs(self) -> int:
        return int(self.seq_lens.shape[0])

    @staticmethod
    def build(seqs_tokens: List[List[int]], seqs_ctx_len: List[int], block_tables: List[List[int]], block_size: int,
              device="cpu", state_slots: Optional[List[int]] = None, has_state: Optional[List[bool]] = None,
              all_logits: bool = False, pad_blocks_to: Optional[int] = None) -> "ForwardBatch":
        """Assemble a batch from python lists.

        ``seqs_tokens[b]`` are the new tokens of sequence ``b``; ``seqs_ctx_len[b]`` tokens are already cached.
        Sequences with exactly one new token and a non-empty context must come first (decodes).
        """
        ids, pos, slots, qsl, sl, li = [], [], [], [0], [], []
        num_dec, seen_prefill = 0, False
        for b, (toks, ctx) in enumerate(zip(seqs_tokens, seqs_ctx_len)):
            n = len(toks)
            if n == 1 and ctx > 0 and not seen_prefill:
                num_dec += 1
            else:
                seen_prefill = True
            bt = block_tables[b]
            for j, t in enumerate(toks):
                p = ctx + j
                ids.append(t)
                pos.append(p)
                slots.append(bt[p // block_size] * block_size + p % block_size)
            qsl.append(qsl[-1] + n)
            sl.append(ctx + n)
            if all_logits:
                li.extend(range(qsl[-2], qsl[-1]))
            else:
                li.append(qsl[-1] - 1)
        maxb = max((len(b) for b in block_tables), default=1)
        if pad_blocks_to:
            maxb = max(maxb, pad_blocks_to)
        bt_t = torch.zeros(len(block_tables), max(1, maxb), dtype=torch.int32)
        for b, bt in enumerate(block_tables):
            if bt:
                bt_t[b, :len(bt)] = torch.tensor(bt, dtype=torch.int32)
        qlens = [qsl[i + 1] - qsl[i] for i in range(len(sl))]
        fb = ForwardBatch(
            input_ids=torch.tensor(ids, dtype=torch.int64, device=device),
            positions=torch.tensor(pos, dtype=torch.int32, device=device),
            slot_mapping=torch.tensor(slots, dtype=torch.int32, device=device),
            block_tables=bt_t.to(device),
            seq_lens=torch.tensor(sl, dtype=torch.int32, device=device),
            query_start_loc=torch.tensor(qsl, dtype=torch.int32, device=device),
            num_decodes=num_dec, max_query_len=max(qlens, default=1), max_seq_len=max(sl, default=0),
            logits_indices=torch.tensor(li, dtype=torch.int64, device=device),
            seq_lens_host=sl, query_lens_host=qlens,
        )
        if state_slots is not None:
            fb.state_slots = torch.tensor(state_slots, dtype=torch.int32, device=device)
            fb.state_slots_host = list(state_slots)
            fb.has_state_host = list(has_state) if has_state is not None else [c > 0 for c in seqs_ctx_len]
        return fb
