"""Worker of tests/test_gpu_ep.py: expert-parallel layer over N GPUs vs the single-GPU layer."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from strata_b200 import MoeContext, MoeLayer, synth
from strata_b200.ep import EpMoe, EpMoePeer, owner_block


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    fmt = int(sys.argv[1])
    T = int(sys.argv[2])
    mode = sys.argv[3] if len(sys.argv) > 3 else "nccl"
    cfg = synth.MoeConfig("ep_gpu", H=512, I=256, E=16, k=4, fmt=fmt, T=T, seed=9,
                          I_shared=128 if fmt == synth.FMT_NVFP4 else 0, zipf_s=1.1)
    B = owner_block(cfg, world)
    ctx = MoeContext(dev.index)
    torch.cuda.set_stream(ctx.stream)
    Tl = T // world
    part = synth.build_layer(cfg, dev, expert_begin=rank * B, expert_end=(rank + 1) * B)
    ml = MoeLayer(ctx, cfg, max_tokens=Tl, expert_begin=rank * B, expert_count=B, max_pairs=T * cfg.k)
    ml.load_synth(part)
    x_local = part.x[rank * Tl:(rank + 1) * Tl].contiguous()
    if mode == "peer":
        ep = EpMoePeer(ml, cfg, rank, world, T * cfg.k, wait_ms=5000)
        for _ in range(3):          # both window parities and a reuse of the first
            out = ep.forward(x_local)
    else:
        ep = EpMoe(ml, cfg, rank, world)
        out = ep.forward(x_local)
    ctx.synchronize()
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    ok = True
    if rank == 0:
        full = synth.build_layer(cfg, dev)
        ref_layer = MoeLayer(ctx, cfg, max_tokens=T)
        ref_layer.load_synth(full)
        ref = ref_layer.forward(full.x)
        ctx.synchronize()
        got = torch.cat(gathered, 0)
        rel = ((got - ref).norm() / ref.norm()).item()
        print(f"ep world={world} mode={mode} fmt={fmt} T={T} rel_l2={rel:.3e}")
        ok = rel <= 2e-3
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.barrier()
    if mode == "peer":
        ep.close()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
