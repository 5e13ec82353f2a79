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
    (strata_moe_ep_*): a token's row is stored straight into the window of every rank that owns one of
    its experts (once per owner) by the dispatch kernel, and each owner's routing-weighted partial sum
    for the token is loaded straight from its window by the combine kernel.  Nothing on the data path
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

    def forward(self, x, out=None, expected_rows=0, join=True):
        return self.state.forward(x, out, expected_rows, join)

    def close(self):
        self.state.close()
        for w in self.windows:
            if not w.owned:
                w.close()
        dist.barrier()
        self.own.close()


class EpMoePeerPipelined:
    """A step cut into token micro-batches that are in flight together: each part has its own context (stream and
    workspaces), its own layer object over the SAME weights (borrowed in place) and its own windows, so the dispatch
    and combine kernels of one part (NVLink copies, a few CTAs' worth of work) run while the expert GEMMs of the other
    occupy the tensor cores.  Results are identical to the one-part step: tokens are independent.

    make_layer(ctx, max_tokens, max_pairs) -> MoeLayer with the rank's weights registered."""

    def __init__(self, make_layer, cfg, rank, world, tokens, row_capacity, parts=2, group=None, wait_ms=0):
        from .api import MoeContext
        self.cfg, self.parts = cfg, []
        dev = torch.cuda.current_device()
        bounds = [tokens * i // parts for i in range(parts + 1)]
        for i in range(parts):
            n = bounds[i + 1] - bounds[i]
            cap = max(1, (row_capacity * n + tokens - 1) // tokens + 1024)
            ctx = MoeContext(dev)
            layer = make_layer(ctx, n, cap)
            self.parts.append((bounds[i], bounds[i + 1], ctx, layer, EpMoePeer(layer, cfg, rank, world, cap, group, wait_ms)))

    def forward(self, x, out=None):
        if out is None:
            out = torch.empty(x.shape[0], self.cfg.H, dtype=torch.float32, device=x.device)
        for a, b, ctx, layer, ep in self.parts:
            ep.forward(x[a:b], out[a:b], join=False)
        for a, b, ctx, layer, ep in self.parts:
            ctx.leave()
        return out

    def synchronize(self):
        for a, b, ctx, layer, ep in self.parts:
            ctx.synchronize()

    def kernel_launches(self):
        return sum(ctx.stats().kernel_launches for a, b, ctx, layer, ep in self.parts)

    def close(self):
        for a, b, ctx, layer, ep in self.parts:
            ep.close()
