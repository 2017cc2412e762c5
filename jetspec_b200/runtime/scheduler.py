"""Continuous-batching scheduler over a :class:`PagedKVPool`.

``step()`` is called once per forward iteration.  It admits waiting requests
first-come-first-served while the batch and the pool have room (evicting a resident
sequence chosen by the eviction policy when the pool is short), and reports the
running batch plus telemetry.  An evicted sequence is checkpointed as its token
lists and re-queued by ``restore_sequence``; it resumes by re-prefilling
``prompt + tokens decoded so far``.

Same responsibilities as ``jetspec/inference_engine/scheduler.py:33-271``.  Two
behaviours differ on purpose: the ``lru`` policy uses the pool's last-use clock
(the reference's uses arrival time), and a checkpoint always keeps the prompt
(the reference drops it for a sequence evicted during decode), so a restored
request is always complete.  Unlike the reference, the engine's batch loops do
drive admission / finish / eviction through this class.
"""
from __future__ import annotations

import random
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from .kv_pool import EvictionFailed, PagedKVPool


@dataclass
class SequenceRequest:
    seq_id: int
    input_ids: list                      # prompt tokens (prefill) or [next token] (decode)
    prompt_len: Optional[int] = None
    arrival_time: float = field(default_factory=time.time)
    priority: float = 0.0                # lower = evicted first under "priority_score"
    max_new_tokens: int = 256
    temperature: float = 0.0
    use_tree: bool = False
    tree_drafter: Optional[object] = None
    tree_accept_fn: Optional[Callable] = None
    output_tokens: list = field(default_factory=list)
    logits_last: Optional[object] = None
    is_prefill: bool = True
    prompt_tokens: list = field(default_factory=list)   # kept for checkpoint / restore
    reserve_tokens: int = 0              # extra slots wanted beyond the prompt (tree window etc.)

    def __post_init__(self):
        if self.prompt_len is None:
            self.prompt_len = len(self.input_ids)
        if not self.prompt_tokens:
            self.prompt_tokens = list(self.input_ids[: self.prompt_len])


@dataclass
class SchedulerOutput:
    admitted: list = field(default_factory=list)
    running: list = field(default_factory=list)
    evicted: list = field(default_factory=list)
    finished: list = field(default_factory=list)
    timestamp: float = field(default_factory=time.time)
    cache_utilization: float = 0.0
    batch_size: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    admission_reason: str = ""           # "prefill" / "decode" / "batched"


class Scheduler:
    def __init__(self, cache: PagedKVPool, max_batch_size: int = 32, prefill_batch_size: int = 8,
                 scheduling_policy: str = "fcfs", eviction_policy: str = "lru", max_queue: Optional[int] = None):
        self.cache = cache
        self.max_batch_size = int(max_batch_size)
        self.prefill_batch_size = int(prefill_batch_size)
        self.policy = scheduling_policy
        self.evict_policy = eviction_policy
        self.max_queue = max_queue
        self.waiting_queue: deque = deque()
        self.running: dict = {}
        self.finished: dict = {}
        self.evicted: dict = {}

    def admit_request(self, req: SequenceRequest) -> bool:
        """Queue a request; False when the queue bound is reached (caller backs off)."""
        if self.max_queue is not None and len(self.waiting_queue) + len(self.running) >= self.max_queue:
            return False
        self.waiting_queue.append(req)
        return True

    def step(self) -> SchedulerOutput:
        out = SchedulerOutput()
        admitted_now = 0
        while (self.waiting_queue and len(self.running) + len(out.admitted) < self.max_batch_size
               and admitted_now < self.prefill_batch_size):
            req = self.waiting_queue[0]
            want = req.prompt_len + req.reserve_tokens
            if not self.cache.admit_sequence(req.seq_id, want):
                break
            before = set(self.cache.resident())
            protect = [r.seq_id for r in out.admitted]
            if not self._feasible_without(req.seq_id, want, protect):
                # only the pages of requests admitted in this very step would make room, and those are never
                # evicted: stop here instead of evicting every other sequence for nothing
                break
            ok = self._allocate_protecting(req.seq_id, want, protect)
            for sid in before - set(self.cache.resident()):
                victim = self.running.pop(sid, None)
                if victim is not None:
                    self.evicted[sid] = self._checkpoint_seq(victim)
                    out.evicted.append(victim)
            if not ok:
                break
            out.admitted.append(self.waiting_queue.popleft())
            admitted_now += 1
        out.running = list(self.running.values()) + out.admitted
        for req in out.admitted:
            self.running[req.seq_id] = req
            req.is_prefill = True
        out.prefill_tokens = sum(r.prompt_len for r in out.admitted)
        out.decode_tokens = sum(1 for r in out.running if not r.is_prefill)
        out.batch_size = len(out.running)
        out.cache_utilization = self._compute_utilization()
        out.admission_reason = ("batched" if out.admitted and out.decode_tokens
                                else "prefill" if out.admitted else "decode")
        return out

    def _feasible_without(self, seq_id: int, want: int, protect: list) -> bool:
        """Could ``want`` positions be granted by evicting only sequences outside ``protect``?"""
        cache = self.cache
        have = len(cache.state(seq_id).pages) if cache.has(seq_id) else 0
        need = cache.pages_for(want) - have
        evictable = sum(len(cache.state(sid).pages) for sid in self.running
                        if sid not in protect and sid != seq_id and cache.has(sid))
        return need <= cache.free_page_count + evictable

    def _allocate_protecting(self, seq_id: int, want: int, protect: list) -> bool:
        """Allocate, evicting policy-chosen victims; never evict a request admitted this step."""
        cache = self.cache
        while not cache.allocate_slots(seq_id, want, allow_evict=False):
            cands = [r for sid, r in self.running.items() if sid not in protect and sid != seq_id
                     and cache.has(sid)]
            victim = self._pick_victim(cands)
            if victim is None:
                if cache.has(seq_id) and not cache.state(seq_id).pages:
                    cache.free(seq_id)
                return False
            cache.evict_sequence(victim.seq_id)
        return True

    def mark_finished(self, seq_id: int) -> None:
        req = self.running.pop(seq_id, None)
        if req is not None:
            self.finished[seq_id] = req
            self.cache.free(seq_id)

    def mark_decode_step(self, seq_id: int, next_token: int, logits=None) -> None:
        req = self.running.get(seq_id)
        if req is None:
            return
        req.output_tokens.append(int(next_token))
        req.input_ids = [int(next_token)]
        req.is_prefill = False
        req.logits_last = logits

    def evict_sequence(self, seq_id: Optional[int] = None) -> Optional[SequenceRequest]:
        victim = (self._pick_victim(list(self.running.values())) if seq_id is None
                  else self.running.get(seq_id))
        if victim is None:
            return None
        try:
            self.cache.evict_sequence(victim.seq_id)
        except EvictionFailed:
            return None
        self.running.pop(victim.seq_id, None)
        self.evicted[victim.seq_id] = self._checkpoint_seq(victim)
        return victim

    def restore_sequence(self, seq_id: int) -> Optional[SequenceRequest]:
        ck = self.evicted.pop(seq_id, None)
        if ck is None:
            return None
        full = list(ck["prompt_tokens"]) + list(ck["output_tokens"])
        req = SequenceRequest(seq_id=seq_id, input_ids=full, prompt_len=len(full),
                              output_tokens=list(ck["output_tokens"]), prompt_tokens=list(ck["prompt_tokens"]),
                              max_new_tokens=ck["max_new_tokens"], temperature=ck["temperature"],
                              priority=ck["priority"], reserve_tokens=ck["reserve_tokens"],
                              use_tree=ck["use_tree"], tree_drafter=ck["tree_drafter"],
                              tree_accept_fn=ck["tree_accept_fn"], arrival_time=ck["arrival_time"])
        self.waiting_queue.append(req)
        return req

    def _pick_victim(self, cands: list) -> Optional[SequenceRequest]:
        if not cands:
            return None
        decoding = [r for r in cands if not r.is_prefill]
        pool = decoding or cands
        if self.evict_policy == "priority_score":
            return min(pool, key=lambda r: r.priority)
        if self.evict_policy == "random":
            return random.choice(pool)
        return min(pool, key=lambda r: self.cache.state(r.seq_id).last_used if self.cache.has(r.seq_id) else 0)

    def _checkpoint_seq(self, req: SequenceRequest) -> dict:
        return {"seq_id": req.seq_id, "prompt_tokens": list(req.prompt_tokens),
                "output_tokens": list(req.output_tokens), "prompt_len": len(req.prompt_tokens),
                "num_decoded": len(req.output_tokens), "max_new_tokens": req.max_new_tokens,
                "temperature": req.temperature, "priority": req.priority, "reserve_tokens": req.reserve_tokens,
                "use_tree": req.use_tree, "tree_drafter": req.tree_drafter, "tree_accept_fn": req.tree_accept_fn,
                "arrival_time": req.arrival_time}

    def _compute_utilization(self) -> float:
        return self.cache.utilization()

    @property
    def has_work(self) -> bool:
        return bool(self.waiting_queue or self.running)
