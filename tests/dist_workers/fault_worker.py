"""Host-side failure scenarios on gloo ranks (no GPU involved).

  --mode exit      rank (world-1) announces that it leaves after step 2 and exits; the others notice before step 3
  --mode stall     rank (world-1) stops beating (sleeps) after step 2; the others notice through the staleness rule
  --mode crash     rank (world-1) dies with an exception after step 2 without announcing it; staleness rule again
  --mode pg        rank (world-1) never joins a collective; the others' all-reduce ends with an error inside the
                   process group's timeout
  --mode ppworld   pipeline_parallel() with a stage count that differs from the world size is refused
Survivors print "rank r: detected ..." and exit 0; a survivor that does not notice exits 1.
"""
import argparse
import datetime
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    timeout = datetime.timedelta(seconds=8 if a.mode == "pg" else 60)
    dist.init_process_group("gloo", timeout=timeout)
    victim = world - 1

    if a.mode == "ppworld":
        from transformers import LlamaConfig, LlamaForCausalLM
        from ipex_llm_b200.parallel.pp import pipeline_parallel
        m = LlamaForCausalLM(LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                                         num_attention_heads=4, vocab_size=256))
        try:
            pipeline_parallel(m, world + 1, torch.float32, device="cpu")
        except RuntimeError as e:
            print(f"rank {rank}: detected stage/world mismatch: {str(e)[:60]}", flush=True)
            dist.barrier()
            return 0
        return 1

    if a.mode == "pg":
        t = torch.ones(4)
        dist.all_reduce(t)                      # everyone joins the first one
        if rank == victim:
            time.sleep(14)                      # ... and the victim never joins the second
            os._exit(0)
        t0 = time.time()
        try:
            dist.all_reduce(t)
        except Exception as e:  # noqa: BLE001 - gloo reports a timeout / connection error
            print(f"rank {rank}: detected stuck collective after {time.time() - t0:.1f} s: {type(e).__name__}", flush=True)
            os._exit(0)
        os._exit(1)

    from ipex_llm_b200.parallel.health import PeerLostError, RankMonitor
    mon = RankMonitor(timeout=3.0)
    dist.barrier()
    for step in range(6):
        # "compute" of the step, then the host-side check that precedes the next launch / collective
        time.sleep(0.2)
        mon.beat(step)
        if rank == victim and step == 2:
            if a.mode == "exit":
                mon.leave("test: planned exit between steps")
                os._exit(0)
            if a.mode == "stall":
                time.sleep(8)
                os._exit(0)
            if a.mode == "crash":
                os._exit(17)
        try:
            mon.wait_for_step(step)
        except PeerLostError as e:
            assert e.ranks == [victim], e.ranks
            assert step >= 2, step
            print(f"rank {rank}: detected {e}", flush=True)
            os._exit(0)
    os._exit(1)


if __name__ == "__main__":
    sys.exit(main())
