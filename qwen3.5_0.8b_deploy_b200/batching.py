"""Continuous batching over the hybrid stack's pools: a queue of requests, admission into free rows between decode
steps, retirement of finished sequences.

The reference stops at the page bookkeeping (``PagedKVCache::allocate_sequence / append_tokens / release_sequence /
shrink_sequence``, src/backend/cuda/kernels/paged_kv.cpp:90-168) and never drives it; this is the loop that does, on
top of ``b200attn_stack_admit / retire / step``.  The policy is first come, first served: before every step, queued
requests are admitted while a row and enough pages are free; a sequence leaves when it has produced its
``max_new_tokens`` or emitted ``eos``.  The backend only needs ``begin_batching, admit, retire, step, read_tokens``,
so the policy is testable without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


@dataclass
class Request:
    rid: int
    prompt: object                 # int32 device tensor (or any sequence for a fake backend)
    max_new_tokens: int
    eos: int | None = None
    tokens: list[int] = field(default_factory=list)     # generated so far


class OutOfCapacity(Exception):
    """Raised by a backend's admit() when rows or pages are exhausted; the request stays queued."""


class ContinuousBatcher:
    def __init__(self, backend, max_rows: int):
        self.backend = backend
        self.max_rows = max_rows
        self.queue: deque[Request] = deque()
        self.rows: list[Request] = []          # rows[r] = request running in row r (dense, as on the device)
        self.finished: list[Request] = []
        self.steps = 0
        backend.begin_batching()

    def submit(self, req: Request) -> None:
        if req.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be > 0")
        self.queue.append(req)

    def _admit_waiting(self) -> None:
        while self.queue and len(self.rows) < self.max_rows:
            req = self.queue[0]
            try:
                row = self.backend.admit(req.prompt, len(req.prompt) + req.max_new_tokens)
            except OutOfCapacity:
                break                           # keep the order: nothing behind the head is admitted before it
            assert row == len(self.rows), "rows are handed out densely"
            self.queue.popleft()
            self.rows.append(req)

    def _finished(self, req: Request) -> bool:
        return len(req.tokens) >= req.max_new_tokens or (req.eos is not None and req.tokens[-1] == req.eos)

    def _take_tokens(self, first_row: int) -> int:
        """Appends the newest token of rows [first_row, active) to their requests and retires the finished ones, highest
        row first (the row that moves into a freed place has then already been looked at).  Returns how many left."""
        toks = self.backend.read_tokens(len(self.rows))
        for r in range(first_row, len(self.rows)):
            self.rows[r].tokens.append(int(toks[r]))
        gone = 0
        for r in reversed(range(first_row, len(self.rows))):
            if self._finished(self.rows[r]):
                self.backend.retire(r)
                self.finished.append(self.rows[r])
                last = self.rows.pop()
                if r < len(self.rows):
                    self.rows[r] = last
                gone += 1
        return gone

    def run(self, max_steps: int = 1 << 30) -> list[Request]:
        """Runs until queue and rows are empty (or max_steps decode steps were taken); returns the finished requests in
        the order they finished."""
        while self.rows or self.queue:
            n_before = len(self.rows)
            self._admit_waiting()
            if len(self.rows) > n_before and self._take_tokens(n_before):
                continue                         # the prompt pass gave the first token; a request that wanted one is gone again
            if not self.rows:
                raise OutOfCapacity("the head of the queue does not fit an empty stack")
            if self.steps >= max_steps:
                break
            self.backend.step()
            self.steps += 1
            self._take_tokens(0)
        return self.finished


class StackBackend:
    """The hybrid stack as a batching backend: every step runs the captured decode graph over all rows."""

    def __init__(self, stack, ops_module):
        import torch
        self.torch = torch
        self.stack = stack
        self.ops = ops_module
        self.n_rows = stack.cfg.max_seqs
        self.captured = False

    def begin_batching(self) -> None:
        self.stack.begin_batching()

    def admit(self, prompt, reserve_tokens: int) -> int:
        try:
            return self.stack.admit(prompt, reserve_tokens)
        except self.ops.B200AttnError as e:
            if e.status == self.ops.ERR_NOMEM:
                raise OutOfCapacity(str(e)) from e
            raise

    def retire(self, row: int) -> None:
        self.stack.retire(row)

    def step(self) -> None:
        if not self.captured:
            self.stack.capture_decode(self.n_rows)     # one graph over all rows: inactive rows (slot -1) are skipped on the device
            self.captured = True
        self.stack.step(self.n_rows)

    def read_tokens(self, n_active: int):
        return self.stack.get_tokens(self.n_rows)[:n_active].cpu().tolist()
