"""Failure detection without touching a GPU: gloo ranks that leave, stall, crash or never join a collective, a
pipeline stage count that does not match the world size, and the request timeout of the HTTP server."""
import asyncio
import os
import subprocess
import sys

import pytest

from tests.test_dist import WORKERS, _free_port


def _run(mode, nproc=3, timeout=120):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(WORKERS, "fault_worker.py"), "--mode", mode]
    e = dict(os.environ)
    e.setdefault("OMP_NUM_THREADS", "2")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.parametrize("mode", ["exit", "stall"])
def test_survivors_notice_a_rank_that_leaves_or_stalls(mode):
    res = _run(mode)
    assert res.stdout.count(": detected lost peer rank(s): 2") == 2, res.stdout[-2000:] + res.stderr[-2000:]


def test_survivors_notice_a_rank_that_crashes():
    res = _run("crash")
    # torchrun tears the job down once it sees the dead child; the survivors may or may not get to print first,
    # but the job must end with an error instead of hanging
    assert res.returncode != 0 or "detected lost peer" in res.stdout


def test_collective_with_a_missing_rank_ends_within_the_group_timeout():
    res = _run("pg", nproc=2, timeout=90)
    assert "detected stuck collective" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_pipeline_stage_count_must_equal_world_size():
    res = _run("ppworld", nproc=2)
    assert res.returncode == 0 and res.stdout.count("detected stage/world mismatch") == 2, \
        res.stdout[-2000:] + res.stderr[-2000:]


def test_rank_monitor_with_a_fake_store_and_clock():
    from ipex_llm_b200.parallel.health import PeerLostError, RankMonitor

    class Store(dict):
        def set(self, k, v):
            self[k] = v

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)

    now = [100.0]
    store = Store()
    m0 = RankMonitor(store, rank=0, world_size=2, timeout=5.0, clock=lambda: now[0])
    m1 = RankMonitor(store, rank=1, world_size=2, timeout=5.0, clock=lambda: now[0])
    m0.check()
    now[0] += 4.0
    m1.beat(0)
    m0.beat(0)
    m0.check()
    now[0] += 6.0                      # rank 1 silent for 6 s > 5 s
    with pytest.raises(PeerLostError) as ei:
        m0.check()
    assert ei.value.ranks == [1] and "no heartbeat" in ei.value.reason[1]
    m1.beat(1)
    m0.check()                         # it came back
    m1.leave("maintenance")
    with pytest.raises(PeerLostError, match="maintenance"):
        m0.check()


def test_http_request_times_out_when_the_worker_produces_nothing(monkeypatch):
    """IPEX_LLM_FASTAPI_TIMEOUT bounds the wait for a request's next piece (reference
    python/llm/src/ipex_llm/serving/fastapi/api_server.py:115)."""
    from fastapi import HTTPException
    from ipex_llm_b200.serving.api_server import FastApp
    monkeypatch.setenv("IPEX_LLM_FASTAPI_TIMEOUT", "0.2")

    class Req:
        def __init__(self):
            self.out = asyncio.Queue()

    class Worker:
        model_name = "fake"
        stats = {"requests": 0, "batches": 0, "generated_tokens": 0, "first_token_s": [], "next_token_s": []}
        waiting = asyncio.Queue()

    app = FastApp(Worker())

    async def go():
        with pytest.raises(HTTPException) as ei:
            await app._collect(Req())
        assert ei.value.status_code == 504

    asyncio.run(go())
