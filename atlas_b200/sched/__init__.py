"""Scheduler: continuous batching, admission, preemption, policies, speculative control."""
from .policy import FifoPolicy, SlaiPolicy, make_policy  # noqa: F401
from .scheduler import Scheduler  # noqa: F401
from .sequence import FinishReason, ScheduledSeq, SchedulerOutput, SeqStatus, Sequence  # noqa: F401
