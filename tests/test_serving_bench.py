"""The closed-loop load tool's own logic, without a GPU: a stand-in engine that answers every
request with a fixed number of tokens after a fixed delay."""
import threading
import time

from firefly_b200.engine.engine import ResultQueue, StepOutput
from firefly_b200.serving_bench import report, run_load


class _FakeEngine:
    def __init__(self, queue, first_s=0.02, token_s=0.002, fail_every=0):
        self.q, self.first_s, self.token_s, self.fail_every = queue, first_s, token_s, fail_every
        self.stats = {"steps": 0}
        self.live = 0
        self.most_live = 0
        self.seen = []
        self._lock = threading.Lock()
        self._threads = []

    def start(self):
        pass

    def stop(self):
        for t in self._threads:
            t.join()

    def async_generate(self, rid, ids, max_tokens, sampling):
        with self._lock:
            self.live += 1
            self.most_live = max(self.most_live, self.live)
            self.seen.append((rid, len(ids), max_tokens, sampling.seed))
            n = len(self.seen)
        t = threading.Thread(target=self._serve, args=(rid, max_tokens, n))
        self._threads.append(t)
        t.start()

    def _serve(self, rid, max_tokens, n):
        time.sleep(self.first_s)
        if self.fail_every and n % self.fail_every == 0:
            with self._lock:
                self.live -= 1
            self.q.push(StepOutput(rid, [], True, "error: made up"))
            return
        for k in range(max_tokens):
            last = k == max_tokens - 1
            if last:
                with self._lock:
                    self.live -= 1
            self.q.push(StepOutput(rid, [k], last, "length" if last else None))
            time.sleep(self.token_s)


def test_closed_loop_keeps_the_concurrency_and_counts_tokens():
    q = ResultQueue()
    eng = _FakeEngine(q)
    prompts = [[1] * (i + 1) for i in range(11)]
    res = run_load(eng, q, prompts, concurrency=3, max_tokens=5)
    assert eng.most_live == 3 and len(eng.seen) == 11
    assert [s[1] for s in eng.seen] == list(range(1, 12))          # in order, each prompt once
    assert res["successful"] == 11 and res["failed"] == 0 and res["total_tokens"] == 55
    assert 0.015 < res["ttft_s"]["median"] < 0.2
    assert 0.001 < res["tpot_s"]["median"] < 0.05
    assert res["tokens_per_s"] > 0 and "P99 TPOT" in report(res)


def test_failed_requests_are_counted_apart():
    q = ResultQueue()
    eng = _FakeEngine(q, fail_every=4)
    res = run_load(eng, q, [[1, 2]] * 8, concurrency=2, max_tokens=3)
    assert res["failed"] == 2 and res["successful"] == 6 and res["total_tokens"] == 18
    assert "Failed Requests:     2" in report(res)
