"""Request / sequence state tracked by the scheduler."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Hashable, List, Optional

from ..sampling import RequestRng, SamplingParams


class SeqStatus(enum.Enum):
    WAITING = "waiting"          # queued, owns nothing
    PREFILL = "prefill"          # admitted, prompt (or resume) chunks still to compute
    RUNNING = "running"          # decoding
    PREEMPTED = "preempted"      # blocks released, will be recomputed on resume
    SWAPPED = "swapped"          # computed KV (and recurrent state) parked in the host tier, resumes without recompute
    FINISHED = "finished"


class FinishReason(str, enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    TIMEOUT = "timeout"
    ERROR = "error"
    TOOL_CALLS = "tool_calls"


@dataclass
class Sequence:
    request_id: str
    prompt_tokens: List[int]
    sampling: SamplingParams
    arrival: float = field(default_factory=time.monotonic)
    namespace: Hashable = 0               # prefix-cache namespace (adapter id, cache salt)
    priority: int = 0
    deadline: Optional[float] = None      # monotonic time after which the request is timed out
    grammar: Any = None
    logits_processors: List[Callable] = field(default_factory=list)
    disable_spec: bool = False
    adapter_slot: int = 0
    # ---- runtime state
    status: SeqStatus = SeqStatus.WAITING
    output_tokens: List[int] = field(default_factory=list)
    blocks: List[int] = field(default_factory=list)
    pinned_nodes: list = field(default_factory=list)
    num_computed: int = 0                 # tokens whose KV / recurrent state is in the cache
    num_cached_tokens: int = 0            # prefix-cache hit length at (last) admission
    state_slot: Optional[int] = None
    has_state: bool = False
    drafts: List[int] = field(default_factory=list)       # pending speculative tokens
    draft_hidden: Any = None
    finish_reason: Optional[FinishReason] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    first_scheduled_time: Optional[float] = None
    num_preemptions: int = 0
    host_blocks: List[int] = field(default_factory=list)  # host-tier blocks while SWAPPED
    host_state: Optional[int] = None
    disk_blocks: List[int] = field(default_factory=list)  # disk-tier records while spilled below the host tier
    logprobs: List[Any] = field(default_factory=list)
    spec_accepted: int = 0
    spec_proposed: int = 0
    rng: RequestRng = None  # type: ignore
    mm: Any = None                        # models.vision.MultiModalInputs of a request with images

    def __post_init__(self):
        if self.rng is None:
            self.rng = RequestRng(self.sampling.seed, self.request_id)

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt_tokens + self.output_tokens

    def token_at(self, pos: int) -> int:
        n = len(self.prompt_tokens)
        return self.prompt_tokens[pos] if pos < n else self.output_tokens[pos - n]

    def tokens_range(self, lo: int, hi: int) -> List[int]:
        """``all_tokens[lo:hi]`` without building the concatenated list."""
        n = len(self.prompt_tokens)
        if hi <= n:
            return self.prompt_tokens[lo:hi]
        if lo >= n:
            return self.output_tokens[lo - n:hi - n]
        return self.prompt_tokens[lo:] + self.output_tokens[:hi - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.output_tokens)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_tokens)

    @property
    def num_uncomputed(self) -> int:
        return self.num_tokens - self.num_computed

    @property
    def finished(self) -> bool:
        return self.status == SeqStatus.FINISHED


@dataclass
class ScheduledSeq:
    seq: Sequence
    start: int            # first token position computed this step
    num_tokens: int       # rows this step
    sample: bool          # the last row produces a token
    is_decode: bool
    verify_drafts: int = 0     # speculative rows included after the real token


@dataclass
class SchedulerOutput:
    items: List[ScheduledSeq] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    restored_snapshots: List[tuple] = field(default_factory=list)   # (snapshot_slot, seq_slot)
    swap_out: List[tuple] = field(default_factory=list)             # (device blocks, host blocks, state slot, host state)
    swap_in: List[tuple] = field(default_factory=list)              # (host blocks, device blocks, host state, state slot)
    disk_out: List[tuple] = field(default_factory=list)             # (host blocks, disk records): spilled before the swap-outs
    disk_in: List[tuple] = field(default_factory=list)              # (disk records, host blocks): staged before the swap-ins
    snapshot_requests: List[tuple] = field(default_factory=list)    # (item index, rows from chunk start, snapshot slot, node)

    @property
    def num_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items)

    @property
    def empty(self) -> bool:
        return not self.items
