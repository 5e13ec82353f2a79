"""Expert parallelism for the MoE layer: one process per GPU, experts sharded by contiguous index
blocks, token rows exchanged with all-to-allv before and after the expert GEMMs.

The reference places experts on several GPUs of ONE process and moves activations through the
host (src/models/glm52/glm_runtime.cpp:650-652, 1561-1576); it has no all-to-all.  Here every
rank owns T/G tokens and E/G experts:

  route (replicated router)        -> ids, weights                        [local kernels]
  group pairs by expert            -> rows sorted by destination rank     [local kernels]
  all-to-all per-expert counts, then all-to-allv of the BF16 rows         [NCCL over NVLink]
  regroup received rows by local expert, grouped expert FFN               [local kernels]
  restore received order, all-to-allv of the fp32 expert outputs back     [NCCL]
  weighted combine in selection-rank order (+ shared expert)              [local kernels]

Received rows always land in local HBM before any kernel reads them; no kernel touches peer
memory.  The compute is delegated to an `ops` object (strata_b200.api.MoeLayer on a GPU; the
CPU tests plug in the oracle) so that the exchange logic itself can be exercised with gloo.
"""
import time

import torch
import torch.distributed as dist


def owner_block(cfg, world):
    assert cfg.E % world == 0, "experts must divide evenly over ranks"
    return cfg.E // world


def exchange(send, send_splits, recv_splits, group=None):
    """all-to-allv of rows (dim 0).  NCCL: all_to_all_single; other backends: point-to-point."""
    out = torch.empty((int(sum(recv_splits)),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(out, send, list(recv_splits), list(send_splits), group=group)
        return out
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    s_off = [0]
    for v in send_splits:
        s_off.append(s_off[-1] + int(v))
    r_off = [0]
    for v in recv_splits:
        r_off.append(r_off[-1] + int(v))
    out[r_off[rank]:r_off[rank + 1]] = send[s_off[rank]:s_off[rank + 1]]
    ops = []
    for peer in range(world):
        if peer == rank:
            continue
        if send_splits[peer]:
            ops.append(dist.P2POp(dist.isend, send[s_off[peer]:s_off[peer + 1]].contiguous(), peer, group))
        if recv_splits[peer]:
            ops.append(dist.P2POp(dist.irecv, out[r_off[peer]:r_off[peer + 1]], peer, group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return out


class EpMoe:
    """One expert-parallel MoE layer on this rank.  `ops` provides route / group / gather_rows /
    experts_grouped / combine with the semantics of strata_b200.api.MoeLayer."""

    def __init__(self, ops, cfg, rank, world, group=None):
        self.ops, self.cfg, self.rank, self.world, self.group = ops, cfg, rank, world, group
        self.block = owner_block(cfg, world)
        self.last = {}

    def forward(self, x):
        cfg, G, B = self.cfg, self.world, self.block
        dev = x.device
        ids, w = self.ops.route(x)
        counts, offsets, perm, inv = self.ops.group(ids, 0, cfg.E, want_inv=True)
        send_rows = self.ops.gather_rows(x, perm, cfg.k)
        # per-expert counts to their owners; the row exchange is sized from them
        counts_mat = counts.view(G, B).contiguous()
        recv_counts = torch.empty_like(counts_mat)
        if dist.get_backend(self.group) == "nccl":
            dist.all_to_all_single(recv_counts, counts_mat, group=self.group)
        else:
            recv_counts = exchange(counts_mat, [1] * G, [1] * G, self.group)
        send_splits = counts_mat.sum(1).cpu().tolist()
        recv_splits = recv_counts.sum(1).cpu().tolist()
        recv_rows = exchange(send_rows, send_splits, recv_splits, self.group)
        n_recv = recv_rows.shape[0]
        # received order is (source rank, local expert, scan order): regroup by local expert
        local_ids = torch.arange(B, device=dev, dtype=torch.int32).repeat(G)
        ids_recv = torch.repeat_interleave(local_ids, recv_counts.reshape(-1).long(), output_size=n_recv)
        lcounts, loffsets, lperm, linv = self.ops.group(ids_recv.view(-1, 1), 0, B, want_inv=True)
        rows_g = self.ops.gather_rows(recv_rows, lperm, 1)
        y_g = self.ops.experts_grouped(rows_g, loffsets)
        y_recv = self.ops.gather_rows(y_g, linv, 1)
        y_back = exchange(y_recv, recv_splits, send_splits, self.group)
        out = self.ops.combine(y_back, inv, w, x if cfg.I_shared else None)
        self.last = dict(ids=ids, weights=w, recv_pairs=n_recv, send_splits=send_splits,
                         recv_splits=recv_splits, local_counts=lcounts)
        return out


class EpMoePeer:
    """The same layer with the exchange done by the library's own kernels over peer memory
    (strata_moe_ep_*): rows are stored straight into the owners' windows by the dispatch kernel and
    expert outputs are loaded straight from them by the combine kernel.  Nothing on the data path
    goes through NCCL or the host; torch.distributed only carries the 64-byte window handles once."""

    def __init__(self, layer, cfg, rank, world, row_capacity, group=None, wait_ms=0):
        from .api import EpState, EpWindow
        self.layer, self.cfg, self.rank, self.world = layer, cfg, rank, world
        ctx = layer.ctx
        self.own, self.windows, self.state, err = None, [], None, None
        try:
            self.own = EpWindow.alloc(ctx, EpWindow.bytes_needed(layer, world, row_capacity))
        except Exception as e:      # still take part in the handle exchange below
            err = e
        handles = [None] * world
        dist.all_gather_object(handles, self.own.handle if self.own else None, group=group)
        try:
            if err is None and any(h is None for h in handles):
                err = RuntimeError("a peer could not allocate its window")
            if err is None:
                self.windows = [self.own if r == rank else EpWindow.open(ctx, handles[r]) for r in range(world)]
                self.state = EpState(layer, rank, world, row_capacity, [w.ptr for w in self.windows], wait_ms)
        except Exception as e:
            err = e
        # agree on the outcome; this is also the barrier after which every window is zeroed and mapped
        ok = torch.tensor([0 if err else 1], device=ctx.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer-memory exchange unavailable: {err or 'a peer failed to map the windows'}")

    def forward(self, x, out=None, expected_rows=0):
        return self.state.forward(x, out, expected_rows)

    def close(self):
        self.state.close()
        for w in self.windows:
            if not w.owned:
                w.close()
        dist.barrier()
        self.own.close()


# ------------------------------------------------------------------------------------------
def bench(args, cfg, T, rank, world, device, peaks, ClockSampler):
    """Multi-GPU leg of bench.py: one layer over `world` ranks, E/world experts per rank.
    Weak scaling (default): T tokens per rank.  Strong scaling (--scaling strong): T tokens in
    total, T/world per rank.  Returns the JSON line dict (rank 0)."""
    import json
    import numpy as np
    from . import MoeContext, MoeLayer, synth

    dist.init_process_group("nccl", device_id=device)
    strong = getattr(args, "scaling", "weak") == "strong"
    if strong:
        assert T % world == 0
        Tl = T // world
    else:
        Tl, T = T, T * world
    B = owner_block(cfg, world)
    ctx = MoeContext(device.index)
    torch.cuda.set_stream(ctx.stream)
    pairs_total = T * cfg.k
    avg = pairs_total // world
    max_pairs = min(pairs_total, max(2 * avg, avg + 4096))
    layer = synth.build_layer(cfg, device, expert_begin=rank * B, expert_end=(rank + 1) * B, T=T)
    x_local = layer.x[rank * Tl:(rank + 1) * Tl].contiguous()
    ml = MoeLayer(ctx, cfg, max_tokens=Tl, expert_begin=rank * B, expert_count=B, max_pairs=max_pairs)
    ml.load_synth(layer)
    exchange_kind = getattr(args, "exchange", "peer")
    exchange_text = None
    if exchange_kind == "peer":
        try:
            ep = EpMoePeer(ml, cfg, rank, world, max_pairs)
            exchange_text = "library kernels over peer memory (NVLink stores / loads, no collective on the data path)"
        except RuntimeError as e:    # every rank raises together; the NCCL exchange is the other GPU path
            exchange_text = f"NCCL all-to-allv (counts, rows, outputs); peer windows failed: {e}"
            ep = EpMoe(ml, cfg, rank, world)
    else:
        ep = EpMoe(ml, cfg, rank, world)
        exchange_text = "NCCL all-to-allv (counts, rows, outputs)"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)

    warm = max(args.warmup, 3)
    for _ in range(warm):
        flush.zero_()
        out = ep.forward(x_local)
    ctx.synchronize()
    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    launches0 = ctx.stats().kernel_launches
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    dist.barrier()
    torch.cuda.synchronize()
    for a, b in evs:
        flush.zero_()
        dist.barrier()
        a.record()
        out = ep.forward(x_local)
        b.record()
    torch.cuda.synchronize()
    dist.barrier()
    launches = ctx.stats().kernel_launches - launches0
    ms = torch.tensor([a.elapsed_time(b) for a, b in evs], device=device, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)           # per step: the slowest rank
    ms_per_step = float(ms.mean())
    ctx.synchronize()    # raises if any step tripped the device status word (overflow, timeout, non-finite)
    ids_loc, _ = ml.route(x_local)
    per_rank = torch.bincount((ids_loc.reshape(-1) // B).long(), minlength=world).double()
    dist.all_reduce(per_rank)     # rows every rank receives in one step
    recv_max = per_rank.max()

    # end to end: pinned host activations in, fp32 result out, every step
    x_host = x_local.cpu().pin_memory()
    out_host = torch.empty(Tl, cfg.H, dtype=torch.float32).pin_memory()
    x_dev = torch.empty_like(x_local)
    e2e = []
    for i in range(args.steps + 2):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        x_dev.copy_(x_host, non_blocking=True)
        o = ep.forward(x_dev)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
        e2e.append(time.perf_counter() - t0)
    e2e_t = torch.tensor(e2e[2:], device=device, dtype=torch.float64)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    if rank == 0:
        t_end = time.perf_counter() + 2.0
    go = torch.ones(1, device=device)
    while True:     # same load until rank 0's clock log has a few samples (all ranks leave together)
        if rank == 0:
            go.fill_(1.0 if (len(sampler.rows) < 6 and time.perf_counter() < t_end) else 0.0)
        dist.broadcast(go, 0)
        if go.item() == 0.0:
            break
        flush.zero_()
        ep.forward(x_local)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ctx.synchronize()
    # where a step's time goes: the four stages of the peer exchange, timed on this rank's stream
    # (each stage's time includes waiting for the slowest peer)
    stage_ms = None
    if isinstance(ep, EpMoePeer):
        st = ep.state
        acc = torch.zeros(4, dtype=torch.float64)
        reps = 5
        for _ in range(reps):
            flush.zero_()
            dist.barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
            ev[0].record()
            st.begin(x_local)
            ev[1].record()
            st.dispatch()
            ev[2].record()
            st.experts()
            ev[3].record()
            st.finish(out)
            ev[4].record()
            torch.cuda.synchronize()
            acc += torch.tensor([ev[i].elapsed_time(ev[i + 1]) for i in range(4)], dtype=torch.float64)
        ctx.synchronize()
        stage_ms = dict(zip(("route_group_publish", "plan_dispatch", "wait_experts_signal", "wait_combine"),
                            [round(float(v), 4) for v in acc / reps]))

    line = None
    if rank == 0:
        flops = 6.0 * cfg.H * cfg.I * pairs_total
        line = {
            "metric": "MoE layer tokens/s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded hash weights, N(0,1) BF16 activations, random-init router)",
            "config": {"workload": f"{cfg.name}: {cfg.description}", "tokens": T, "tokens_per_rank": Tl,
                       "hidden": cfg.H, "intermediate": cfg.I, "experts": cfg.E, "experts_per_rank": B,
                       "top_k": cfg.k, "format": ["mxfp4", "nvfp4", "int4g128"][cfg.fmt],
                       "parallelism": f"ep{world}", "exchange": exchange_text,
                       "l2": "512 MiB buffer rewritten between timed iterations"},
            "roofline": {"bound": "tensor", "achieved": flops / (ms_per_step * 1e-3) / 1e12 / world,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": flops / (ms_per_step * 1e-3) / 1e12 / world / peaks["bf16_tflops"],
                         "traffic": None, "kernel": "whole step per rank (expert GEMMs + exchange)",
                         "peak_source": peaks["source"]},
            "max_rank_pairs": int(recv_max.item()), "mean_rank_pairs": pairs_total / world,
            "e2e": {"value": T / float(e2e_t.mean()), "unit": "tokens/s",
                    "h2d_bytes_per_step": Tl * cfg.H * 2, "d2h_bytes_per_step": Tl * cfg.H * 4},
            "gpu_launches": int(launches),
            "stage_ms_rank0": stage_ms,
            "clocks": clocks,
        }
    dist.barrier()
    dist.destroy_process_group()
    return line
