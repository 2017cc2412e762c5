"""Runtime substrate: paged KV pool, scheduler, attention metadata."""
from .kv_pool import PagedKVPool, SeqState, EvictionRequired, EvictionFailed
from .scheduler import Scheduler, SequenceRequest, SchedulerOutput
from .attn_metadata import AttnMeta, build_attn_metadata

__all__ = ["PagedKVPool", "SeqState", "EvictionRequired", "EvictionFailed", "Scheduler",
           "SequenceRequest", "SchedulerOutput", "AttnMeta", "build_attn_metadata"]
