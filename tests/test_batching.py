"""CPU: the continuous-batching policy (queue, admission into free rows, retirement, dense rows) against a fake backend
that mirrors the stack's row bookkeeping: rows stay dense, the last row moves into a freed place, capacity is counted in
rows and in pages."""
import pytest

import __graft_entry__ as entry


class FakeBackend:
    """Token of request `rid` at position p is rid * 1000 + p; a row remembers which request runs in it."""

    def __init__(self, max_rows, pages):
        self.max_rows, self.pages_free = max_rows, pages
        self.rows = []            # per row: [rid, tokens produced, pages held]
        self.log = []

    def begin_batching(self):
        self.rows.clear()

    def admit(self, prompt, reserve_tokens):
        from qwen35_deploy_b200.batching import OutOfCapacity
        need = -(-reserve_tokens // 64)
        if len(self.rows) >= self.max_rows or need > self.pages_free:
            raise OutOfCapacity("full")
        self.pages_free -= need
        self.rows.append([prompt[0], 1, need])     # the prompt pass yields the first token
        self.log.append(("admit", prompt[0], len(self.rows) - 1))
        return len(self.rows) - 1

    def retire(self, row):
        self.pages_free += self.rows[row][2]
        self.log.append(("retire", self.rows[row][0], row))
        last = self.rows.pop()
        if row < len(self.rows):
            self.rows[row] = last

    def step(self):
        for r in self.rows:
            r[1] += 1

    def read_tokens(self, n_active):
        assert n_active == len(self.rows)
        return [r[0] * 1000 + r[1] - 1 for r in self.rows]


@pytest.fixture()
def batching():
    entry.load_package()
    import importlib
    return importlib.import_module(entry.PKG_NAME + ".batching")


def test_every_request_gets_its_own_tokens_in_order(batching):
    be = FakeBackend(max_rows=3, pages=100)
    cb = batching.ContinuousBatcher(be, max_rows=3)
    lengths = [5, 1, 9, 3, 3, 7, 2]
    for rid, n in enumerate(lengths, start=1):
        cb.submit(batching.Request(rid, [rid] * 10, n))
    done = cb.run()
    assert sorted(r.rid for r in done) == list(range(1, len(lengths) + 1))
    for r in done:
        assert r.tokens == [r.rid * 1000 + p for p in range(lengths[r.rid - 1])], r
    assert not cb.rows and not cb.queue and be.pages_free == 100
    assert max(row for kind, _, row in be.log if kind == "admit") <= 2          # never more than three rows
    admits = [rid for kind, rid, _ in be.log if kind == "admit"]
    assert admits == sorted(admits)                                             # first come, first served


def test_page_budget_holds_back_the_head_of_the_queue(batching):
    be = FakeBackend(max_rows=4, pages=4)             # rows are free, pages are not
    cb = batching.ContinuousBatcher(be, max_rows=4)
    cb.submit(batching.Request(1, [1] * 100, 60))     # 160 tokens = 3 pages
    cb.submit(batching.Request(2, [2] * 100, 60))     # must wait for request 1
    cb.submit(batching.Request(3, [3] * 10, 4))       # would fit, but may not overtake request 2
    done = cb.run()
    assert [r.rid for r in done] == [1, 3, 2] or [r.rid for r in done] == [1, 2, 3]
    order = [(kind, rid) for kind, rid, _ in be.log]
    assert order.index(("retire", 1)) < order.index(("admit", 2)) < order.index(("admit", 3))


def test_eos_ends_a_sequence_early_and_oversized_heads_raise(batching):
    be = FakeBackend(max_rows=2, pages=10)
    cb = batching.ContinuousBatcher(be, max_rows=2)
    cb.submit(batching.Request(7, [7] * 4, 50, eos=7003))
    done = cb.run()
    assert done[0].tokens == [7000, 7001, 7002, 7003]
    cb.submit(batching.Request(8, [8] * 64, 64 * 20))                  # needs 21 pages, the pool has 10
    with pytest.raises(batching.OutOfCapacity):
        cb.run()
    with pytest.raises(ValueError):
        cb.submit(batching.Request(9, [9], 0))
