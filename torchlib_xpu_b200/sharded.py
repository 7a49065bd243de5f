"""Table-wise sharding of TBE across the GPUs of one node: one process per GPU.

Rank r owns T_local tables and looks them up for the WHOLE global batch of B bags; every rank ends
up with the pooled rows of its own slice of the batch (B / G bags) for ALL tables:

    pooled[r] : [B / G, G * D_local]     columns [s*D_local, (s+1)*D_local) come from rank s

(with tables dealt round-robin, global table id = local_table * G + rank). The exchange is not a
separate collective on the forward path: b200tbe_forward writes each pooled vector straight into the
destination rank's receive buffer through its peer mapping (plain 16-byte stores over NVLink), and a
stream-ordered barrier closes the step. On the way back each rank stores the column blocks of its
gradient rows into the owning ranks' matrices with b200tbe_exchange_push, then runs the local fused
backward.

`layout_*` below are pure index arithmetic and are what the CPU (gloo) tests exercise;
`reference_exchange` / `reference_gradient_exchange` are the same data movements as plain
all_to_all_single calls (NCCL on GPUs, gloo on CPU): what the fused paths are compared with.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def owner_of_table(global_table: int, world: int) -> int:
    return global_table % world


def local_tables(rank: int, world: int, total_tables: int) -> list[int]:
    """Global ids of the tables rank holds, in its local order."""
    return list(range(rank, total_tables, world))


def layout_pooled_columns(rank_of_source: int, local_D: int) -> tuple[int, int]:
    """Column range, in a receive buffer, of the pooled rows produced by one source rank."""
    return rank_of_source * local_D, (rank_of_source + 1) * local_D


def layout_batch_rows(rank: int, world: int, B: int) -> tuple[int, int]:
    """Global bags whose pooled rows rank receives."""
    if B % world != 0:
        raise ValueError("global batch %d is not divisible by world size %d" % (B, world))
    per = B // world
    return rank * per, (rank + 1) * per


def reference_exchange(pooled_local: torch.Tensor, group=None) -> torch.Tensor:
    """[B, D_local] on every rank -> [B / G, G * D_local] on every rank, by all_to_all_single."""
    world = dist.get_world_size(group)
    B, local_D = pooled_local.shape
    per = B // world
    recv = torch.empty((world, per, local_D), dtype=pooled_local.dtype, device=pooled_local.device)
    dist.all_to_all_single(recv, pooled_local.contiguous().view(world, per, local_D), group=group)
    return recv.permute(1, 0, 2).reshape(per, world * local_D)


def reference_gradient_exchange(grad_slice: torch.Tensor, group=None) -> torch.Tensor:
    """[B / G, G * D_local] on every rank -> [B, D_local] on every rank (the transpose of the above)."""
    world = dist.get_world_size(group)
    per, total = grad_slice.shape
    local_D = total // world
    send = grad_slice.view(per, world, local_D).permute(1, 0, 2).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(world * per, local_D)


class PooledExchange:
    """Peer-mapped receive / gradient buffers and the fused exchange for one rank (CUDA only)."""

    def __init__(self, rank: int, world: int, B: int, local_D: int, dtype=torch.float16):
        import torch.distributed._symmetric_memory as symm_mem

        if world > 16:
            raise ValueError("at most 16 destinations")
        self.rank, self.world, self.B, self.local_D = rank, world, B, local_D
        self.per = layout_batch_rows(rank, world, B)[1] - layout_batch_rows(rank, world, B)[0]
        self.dtype = dtype
        dev = torch.device("cuda", torch.cuda.current_device())
        # what this rank receives in the forward, and the gradient it hands back in the backward
        self.recv = symm_mem.empty((self.per, world * local_D), dtype=dtype, device=dev)
        self.grad_slice = torch.empty((self.per, world * local_D), dtype=dtype, device=dev)
        self._recv_hdl = symm_mem.rendezvous(self.recv, dist.group.WORLD)
        self.recv_ptrs = [int(p) for p in self._recv_hdl.buffer_ptrs]
        # this rank's column block of every rank's gradients; the peers store into it
        self.grad_local = symm_mem.empty((B, local_D), dtype=dtype, device=dev)
        self._gradl_hdl = symm_mem.rendezvous(self.grad_local, dist.group.WORLD)
        self.gradl_ptrs = [int(p) for p in self._gradl_hdl.buffer_ptrs]
        self._token = torch.zeros(1, device=dev)
        gen = torch.Generator(device=dev).manual_seed(4242 + rank)
        self.grad_slice.copy_(torch.randn((self.per, world * local_D), device=dev, generator=gen).to(dtype))
        self.barrier()

    def barrier(self):
        """Stream-ordered barrier across ranks: everything enqueued before it on every rank has
        finished before anything enqueued after it on any rank starts."""
        dist.all_reduce(self._token)

    def forward_lookup(self, step):
        """Lookup of this rank's tables for the whole batch, pooled vectors written directly into
        the owning ranks' receive buffers."""
        from . import cabi

        cabi.forward(step.weights, step.weights_offsets, step.D_offsets, step.total_D, step.D,
                     step.indices, step.offsets, step.B, outputs=self.recv_ptrs,
                     output_stride=self.world * self.local_D,
                     output_col_offset=self.rank * self.local_D, rows_per_dest=self.per,
                     output_dtype=self.dtype)
        self.barrier()

    def push_gradients(self):
        """Stores every owner's column block of this rank's gradient rows into that owner's matrix
        (b200tbe_exchange_push: NVLink stores stream). No barrier: the caller orders it."""
        from . import cabi

        esz = self.grad_slice.element_size()
        cabi.exchange_push(self.grad_slice, self.gradl_ptrs, self.local_D * esz, self.rank * self.per,
                           self.local_D * esz)

    def gather_gradients(self, step=None):
        """Brings this rank's column block of every rank's gradient matrix into [B, local_D]. The call
        must follow a barrier that follows the previous reader of grad_local on every rank (the
        forward's barrier does), and ends with one."""
        self.push_gradients()
        self.barrier()
        return self.grad_local

    def gather_gradients_async(self, step):
        """The same exchange on a side stream: returns ([B, local_D], event). The event fires when the
        exchange and its barrier are done; pass it to cabi.backward(grad_ready_event=...) and it
        overlaps the linearise + sort part of the backward, which needs only the indices."""
        main = torch.cuda.current_stream()
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream()
        start, ready = torch.cuda.Event(), torch.cuda.Event()
        start.record(main)                     # the peers' gradients are complete in main-stream order
        self._side.wait_event(start)
        with torch.cuda.stream(self._side):
            self.gather_gradients(step)
            ready.record(self._side)
        return self.grad_local, ready

    def launches_per_step(self) -> int:
        return 1  # the gradient push kernel (the forward scatter is part of the lookup kernel)

    def describe(self) -> str:
        return ("pooled rows stored by the lookup kernel into peer receive buffers (NVLink P2P "
                "stores); gradient blocks pushed to their owners by one copy kernel; NCCL all-reduce of "
                "one element as the barrier after each; the push runs on a side stream under the "
                "backward's linearise + sort")


# ---- input distribution: data-parallel batches -> table-wise layout ------------------------------
def destination_major_tables(world: int, total_tables: int) -> list[int]:
    """Global table ids ordered by owning rank, each rank's tables in its local order."""
    return [t for d in range(world) for t in local_tables(d, world, total_tables)]


def _exclusive_offsets(lengths_flat: torch.Tensor) -> torch.Tensor:
    off = torch.zeros(lengths_flat.numel() + 1, dtype=torch.int64, device=lengths_flat.device)
    torch.cumsum(lengths_flat, 0, out=off[1:])
    return off


def kernel_permute_segments(values, lengths_flat, perm):
    """The same through b200tbe_permute_segments (CUDA tensors only)."""
    from . import cabi

    if not values.is_cuda:
        raise RuntimeError("kernel_permute_segments needs CUDA tensors; there is no CPU path")
    lengths_flat = lengths_flat.to(torch.int64)
    perm = perm.to(torch.int64)
    in_off = _exclusive_offsets(lengths_flat)
    out_off = _exclusive_offsets(lengths_flat[perm])
    return cabi.permute_segments(values.contiguous(), in_off, out_off, perm)


def _distribute(lengths_dp, indices_dp, weights_dp, group, permute):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T_global, per = lengths_dp.shape
    if T_global % world != 0:
        raise ValueError("%d tables cannot be dealt to %d ranks evenly" % (T_global, world))
    T_local = T_global // world
    dev = lengths_dp.device
    lengths_dp = lengths_dp.to(torch.int64)
    order = torch.tensor(destination_major_tables(world, T_global), dtype=torch.int64, device=dev)
    # 1. this rank's ids regrouped by destination rank (whole tables move as segments)
    table_len = lengths_dp.sum(1)
    send_lengths = lengths_dp[order].contiguous()
    send = [permute(indices_dp, table_len, order)]
    if weights_dp is not None:
        send.append(permute(weights_dp, table_len, order))
    # 2. bag lengths first: they say how many ids each peer will send
    recv_lengths = torch.empty_like(send_lengths)
    dist.all_to_all_single(recv_lengths, send_lengths, group=group)
    send_splits = table_len[order].view(world, T_local).sum(1).tolist()
    recv_splits = recv_lengths.view(world, T_local * per).sum(1).tolist()
    recv = []
    for buf in send:
        got = torch.empty(int(sum(recv_splits)), dtype=buf.dtype, device=dev)
        dist.all_to_all_single(got, buf, recv_splits, send_splits, group=group)
        recv.append(got)
    # 3. received as (source rank, local table, sample); the lookup wants (local table, global sample)
    seg = torch.arange(world * T_local * per, device=dev).view(world, T_local, per)
    perm = seg.permute(1, 0, 2).reshape(-1)
    lengths_tw = recv_lengths.view(world, T_local, per).permute(1, 0, 2).reshape(T_local, world * per)
    flat = recv_lengths.view(-1)
    indices_tw = permute(recv[0], flat, perm)
    weights_tw = permute(recv[1], flat, perm) if weights_dp is not None else None
    offsets_tw = _exclusive_offsets(lengths_tw.reshape(-1))
    return lengths_tw, offsets_tw, indices_tw, weights_tw


def distribute_inputs(lengths_dp, indices_dp, weights_dp=None, group=None, permute=None):
    """From the data-parallel layout to the table-wise one (CUDA tensors, NCCL).

    lengths_dp [T_global, B / G]: bag lengths of this rank's slice of the global batch for every
    table; indices_dp (and optional per-sample weights_dp): the ids in table-major, sample-minor
    order. Returns, for the tables this rank owns and ALL B samples: lengths [T_local, B], offsets
    [T_local * B + 1], ids and weights in bag order: the arguments of b200tbe_forward /
    b200tbe_backward. Two all_to_all_single calls (lengths, then ids with the sizes the lengths
    announce; one host read of the split sizes in between) and two segment permutations by
    b200tbe_permute_segments. `permute(values, lengths, perm)` replaces the kernel in tests that run
    the collective logic on CPU ranks with a checker's permutation."""
    return _distribute(lengths_dp, indices_dp, weights_dp, group, permute or kernel_permute_segments)
