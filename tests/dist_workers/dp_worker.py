"""Data-parallel optimizer worker: every rank feeds its own gradients to ``FusedLoraAdamW``; after each step all
ranks must hold the parameters that single-process ``torch.optim.AdamW`` reaches on the rank-averaged gradients.
``--device cpu`` exercises the host restatement on gloo ranks, ``--device cuda`` the fused peer-memory kernel."""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    from ipex_llm_b200.parallel.dp import FusedLoraAdamW

    dtype = torch.bfloat16 if cuda else torch.float32
    torch.manual_seed(0)                               # same initial parameters everywhere
    shapes = [(8, 4096), (4096, 8), (8, 11008), (11008, 8), (3, 5)]
    params = [torch.nn.Parameter((torch.randn(s) * 0.1).to(dtype).to(dev)) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    # clipping by the global norm of the averaged gradient, as torch's clip_grad_norm_ on the reference copy
    clip = 0.5
    opt = FusedLoraAdamW(params, lr=1e-2, weight_decay=0.05, max_grad_norm=clip)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.05)
    for step in range(4):
        for p, r in zip(params, ref):
            g = torch.Generator().manual_seed(1000 * step + 10 * rank + p.numel() % 7)
            local = (torch.randn(p.shape, generator=g) * 0.5).to(dtype)
            p.grad.copy_(local.to(dev))
            # reference: mean over ranks of the same (dtype-rounded) gradients
            acc = torch.zeros(p.shape)
            for rr in range(world):
                gg = torch.Generator().manual_seed(1000 * step + 10 * rr + p.numel() % 7)
                acc += (torch.randn(p.shape, generator=gg) * 0.5).to(dtype).float()
            r.grad = (acc / world).to(r.device)
        torch.nn.utils.clip_grad_norm_(ref, clip)
        opt.step()
        ropt.step()
        opt.zero_grad()
        if cuda:
            torch.cuda.synchronize()
            from ipex_llm_b200.ops import cuda_ops
            cuda_ops.check_error_flag(dev)
    tol = 2e-2 if cuda else 1e-6                       # bf16 parameters: one rounding per step
    for p, r in zip(params, ref):
        err = (p.detach().float().cpu() - r.detach().cpu()).abs().max().item()
        assert err <= tol * max(1.0, r.abs().max().item()), (tuple(p.shape), err)
    # every rank holds identical parameters
    flat = opt.flat_params.float()
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi), "ranks diverged"
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: ok")


if __name__ == "__main__":
    main()
