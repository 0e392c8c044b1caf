"""Parallel layer on CPU: two gloo ranks through the real launcher."""

import time

import pytest

from kohakumosstrainer_b200.parallel import selftest


def test_reducer_sums_and_views(tmp_path):
    res = selftest.spawn_results(selftest.reducer_worker, 2, str(tmp_path), ("torch", "fp32"))
    for r in res:
        assert r["views"] and r["same_after_broadcast"] and r["ranks_agree"]
        assert r["rel_err"] < 1e-5
        assert r["buckets"] >= 2 and r["backend"] == "torch"


def test_store_gates(tmp_path):
    res = selftest.spawn_results(selftest.gates_worker, 2, str(tmp_path))
    assert all(r["value"] == {"seed": 1234, "who": "rank0"} for r in res)
    assert all(r["agree"] is False for r in res)  # rank 1 reported a failed write


def test_fail_fast_when_a_rank_raises(tmp_path):
    t0 = time.time()
    with pytest.raises(RuntimeError, match="injected failure on the host"):
        selftest.spawn_results(selftest.raise_worker, 2, str(tmp_path), timeout_s=600)
    assert time.time() - t0 < 30  # the waiting rank was killed, not waited for
