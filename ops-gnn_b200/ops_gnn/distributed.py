"""Row-sharded CSR SpMM over the GPUs of one node (one process per GPU, ``torch.distributed`` for the plumbing).

The reference is a single-device library (no collective appears anywhere in it); this module is the multi-GPU form of
its SpMM path.  Output rows are independent, so the graph is cut into contiguous row ranges that hold equal numbers of
edges (equal rows would leave the first shard of a power-law graph with most of the work).  Every rank owns one such
range of the CSR structure and an equal block of the rows of the dense operand ``X``, as a GNN layer would hold them.
One step is: all-gather the blocks of ``X`` into this GPU's own memory, then run the local SpMM over the rank's rows.

Peer memory: no load anywhere in this module is a multicast load, and NVLS / multicast binding is switched off for
the symmetric-memory buffers.  The NCCL forms land remote rows in the rank's own HBM before the SpMM reads them.  The
``pull`` and ``push`` transports hand a peer's symmetric-memory block to this library's own gather kernel, as its
source (``pull``: plain peer loads) or as its destination (``push``: plain peer stores); the ``copy`` transport
writes into a peer's block with ``cudaMemcpyAsync`` (a copy-engine transfer from this GPU's memory, not a kernel).  No
library kernel of anybody else is ever given a peer pointer.

``feature_chunks > 1`` splits ``X`` by columns into contiguous chunk-major blocks: the all-gather of chunk ``c + 1``
runs on a side stream while the SpMM of chunk ``c`` computes, so the transfer hides behind the math tile by tile.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch


def balanced_row_bounds(rowptr: torch.Tensor, parts: int, row_cost: float = 0.0) -> List[int]:
    """``parts + 1`` row boundaries such that every range ``[b[k], b[k+1])`` holds an equal share of the work.

    Work is ``edges + row_cost * rows``: with ``row_cost = 0`` the ranges hold ``nnz / parts`` edges each; for an SpMM
    use ``row_cost = 1`` (writing one output row moves as many bytes as gathering one row of the dense operand), so a
    shard of many short rows is not handed as many edges as a shard of few hub rows.
    """
    if parts < 1:
        raise ValueError("parts must be positive")
    if row_cost < 0:
        raise ValueError("row_cost must not be negative")
    rows = rowptr.numel() - 1
    work = rowptr.contiguous()
    if row_cost:
        work = work.to(torch.float64) + row_cost * torch.arange(rows + 1, dtype=torch.float64, device=rowptr.device)
    total = float(work[-1]) if rows >= 0 and work.numel() else 0.0
    targets = torch.tensor([total * k / parts for k in range(parts + 1)], dtype=torch.float64, device=rowptr.device)
    if not row_cost:
        targets = torch.tensor([int(total) * k // parts for k in range(parts + 1)], dtype=rowptr.dtype,
                               device=rowptr.device)
    bounds = torch.searchsorted(work, targets.to(work.dtype), right=False).tolist()
    bounds[0], bounds[-1] = 0, rows
    for k in range(1, parts + 1):  # keep the boundaries ordered when many rows are empty
        bounds[k] = min(max(bounds[k], bounds[k - 1]), rows)
    return bounds


def high_priority_group(ranks: Optional[Sequence[int]] = None):
    """A NCCL process group whose collectives are launched on a high-priority stream.

    The staged exchange runs its all-to-alls beside the SpMM of an earlier stage.  The thread blocks of a collective
    launched at default priority are handed out only once every block of the product launched before it has been, so
    the exchange would start when that product is nearly over; at high priority they take the next slots that free up.
    """
    import torch.distributed as dist

    options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    return dist.new_group(ranks=None if ranks is None else list(ranks), backend="nccl", pg_options=options)


def shard_csr(rowptr: torch.Tensor, col: torch.Tensor, value: Optional[torch.Tensor], first: int,
              last: int) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """CSR slice of rows ``[first, last)`` with the pointers rebased to zero; columns stay global."""
    lo, hi = int(rowptr[first]), int(rowptr[last])
    local_ptr = (rowptr[first:last + 1] - lo).clone()
    local_val = None if value is None else value[lo:hi].clone()
    return local_ptr, col[lo:hi].clone(), local_val


class RowShardedSpmm:
    """One rank's share of ``out = A @ X`` (sum reduction) with ``A`` row-sharded and ``X`` block-distributed.

    ``rowptr / col / value`` are the rank's CSR slice (:func:`shard_csr`); ``block_rows`` is the number of rows of
    ``X`` each rank owns (``N / world``); ``local_spmm(ptr, col, value, x)`` runs the local product (default: the
    CUDA ``csr_spmm``; the CPU tests pass a stand-in because the product itself has no CPU path).
    """

    def __init__(self, rowptr, col, value, block_rows: int, feat: int, dtype, device, group=None,
                 local_spmm: Optional[Callable] = None, feature_chunks: int = 1):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rowptr, self.col, self.value = rowptr, col, value
        if feat % feature_chunks != 0:
            raise ValueError("feature_chunks must divide the feature width")
        self.chunks = feature_chunks
        self.chunk_width = feat // feature_chunks
        self.block_rows = block_rows
        # chunk-major gather buffers: chunk c of the full matrix is a contiguous [N, feat / chunks] tensor
        self.gathered = [torch.empty((block_rows * self.world, self.chunk_width), dtype=dtype, device=device)
                         for _ in range(feature_chunks)]
        if local_spmm is None:
            from .torch_sparse_spmm import _native

            out_code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
            local_spmm = lambda ptr, c, v, x: _native.forward(ptr, c, v, x, 0, out_code)[0]  # noqa: E731
        self.local_spmm = local_spmm
        self.side_stream = torch.cuda.Stream(device) if device.type == "cuda" and feature_chunks > 1 else None

    def split_block(self, x_block: torch.Tensor) -> Sequence[torch.Tensor]:
        """Chunk-major copy of a rank's ``[block_rows, feat]`` block (done once, outside the step)."""
        if self.chunks == 1:
            return [x_block.contiguous()]
        return [part.contiguous() for part in x_block.split(self.chunk_width, dim=1)]

    def _gather(self, chunk: int, block_chunk: torch.Tensor) -> None:
        self.dist.all_gather_into_tensor(self.gathered[chunk], block_chunk, group=self.group)

    def __call__(self, block_chunks: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """Run one step; returns the rank's output rows as one ``[rows, feat / chunks]`` tensor per chunk."""
        outputs = []
        if self.side_stream is None:
            for c, block in enumerate(block_chunks):
                self._gather(c, block)
                outputs.append(self.local_spmm(self.rowptr, self.col, self.value, self.gathered[c]))
            return outputs
        main = torch.cuda.current_stream()
        ready = []
        self.side_stream.wait_stream(main)
        with torch.cuda.stream(self.side_stream):
            for c, block in enumerate(block_chunks):
                self._gather(c, block)
                event = torch.cuda.Event()
                event.record(self.side_stream)
                ready.append(event)
        for c in range(self.chunks):
            main.wait_event(ready[c])
            outputs.append(self.local_spmm(self.rowptr, self.col, self.value, self.gathered[c]))
        self.side_stream.wait_stream(main)
        return outputs


class HaloShardedSpmm:
    """One rank's share of ``out = A @ X`` that moves only the rows of ``X`` its shard references.

    ``A`` is cut into the row ranges ``bounds`` (one per rank) and ``X`` is owned by the same ranges, the layout a
    stack of GNN layers produces: a rank's output rows are its block of the next layer's input.  An all-gather
    would hand every rank all of ``X``; a shard of a sparse graph reads far fewer distinct rows than that.  Here the
    set-up (once per graph) finds the distinct columns of the shard, tells every owner which of its rows are wanted,
    and relabels the shard's columns into a compact buffer ``[own rows | halo rows grouped by owner]``.  A step is
    then: pack the wanted rows per peer, one all-to-all with uneven splits that lands the halo in this GPU's memory,
    and the local SpMM over the compact buffer (every kernel reads local memory only in this form).

    ``gather_rows(x, index)`` packs rows (default: the CSR engine run as a gather, a unit pointer array with the
    wanted rows as columns); ``local_spmm`` as in :class:`RowShardedSpmm`.

    ``transport="pull"`` (CUDA only) drops the pack and the all-to-all: the compact buffers live in symmetric memory
    (``torch.distributed._symmetric_memory``, every peer's buffer mapped into this process), and a step runs the
    gather kernel once per peer with the PEER's block as its source and this rank's halo slice as its destination,
    so each wanted row crosses NVLink once, read by plain (non-multicast) loads of the kernel that also writes it into
    place.  Two stream-ordered NCCL barriers bracket the pulls: blocks are complete before anyone reads them, and
    nobody's block changes while a peer still reads it.
    """

    def __init__(self, rowptr, col, value, bounds: Sequence[int], feat: int, dtype, device, group=None,
                 local_spmm: Optional[Callable] = None, gather_rows: Optional[Callable] = None,
                 transport: str = "alltoall"):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if len(bounds) != self.world + 1:
            raise ValueError("bounds must hold one row range per rank")
        self.bounds = [int(b) for b in bounds]
        self.own_first, own_last = self.bounds[self.rank], self.bounds[self.rank + 1]
        self.own_rows = own_last - self.own_first
        edges = torch.tensor(self.bounds, dtype=col.dtype, device=device)

        # distinct columns of the shard, split into the part this rank owns and the halo, grouped by owner
        needed = torch.unique(col)
        owner = torch.searchsorted(edges, needed, right=True) - 1
        remote = needed[owner != self.rank]                      # sorted, hence already grouped by owner
        want_counts = torch.bincount(owner[owner != self.rank], minlength=self.world)
        give_counts = torch.empty_like(want_counts)
        dist.all_to_all_single(give_counts, want_counts, group=group)
        self.want_splits = [int(c) for c in want_counts.tolist()]
        self.give_splits = [int(c) for c in give_counts.tolist()]
        wanted_of_me = torch.empty(sum(self.give_splits), dtype=col.dtype, device=device)
        dist.all_to_all_single(wanted_of_me, remote.contiguous(), self.give_splits, self.want_splits, group=group)
        self.send_rows = (wanted_of_me - self.own_first).contiguous()   # offsets into this rank's block, per peer
        if self.send_rows.numel() and (int(self.send_rows.min()) < 0 or int(self.send_rows.max()) >= self.own_rows):
            raise RuntimeError("a peer asked for rows outside this rank's block: shard bounds disagree between ranks")
        self.halo_rows = int(remote.numel())

        # compact column ids: own rows first, then the halo in the order it is received
        is_own = (col >= self.own_first) & (col < own_last)
        compact = torch.where(is_own, col - self.own_first, self.own_rows + torch.searchsorted(remote, col))
        self.rowptr, self.col, self.value = rowptr, compact.contiguous(), value
        if transport not in ("alltoall", "pull"):
            raise ValueError("transport must be 'alltoall' or 'pull'")
        self.transport = transport
        total_rows = self.own_rows + self.halo_rows
        if transport == "pull":
            self._setup_pull(remote, total_rows, feat, dtype, device)
        else:
            self.compact = torch.empty((total_rows, feat), dtype=dtype, device=device)
        self.own_block = self.compact[:self.own_rows]            # the caller may produce its block here directly
        self.halo = self.compact[self.own_rows:]
        self.unit_ptr = torch.arange(self.send_rows.numel() + 1, dtype=col.dtype, device=device)
        if local_spmm is None or gather_rows is None:
            from .torch_sparse_spmm import _native

            out_code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
            if local_spmm is None:
                local_spmm = lambda ptr, c, v, x: _native.forward(ptr, c, v, x, 0, out_code)[0]  # noqa: E731
            if gather_rows is None:
                gather_rows = lambda x, index: _native.forward(self.unit_ptr, index, None, x, 0, out_code)[0]  # noqa: E731
        self.local_spmm, self.gather_rows = local_spmm, gather_rows

    def _setup_pull(self, remote, total_rows, feat, dtype, device) -> None:
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads only, no multicast binding
        import torch.distributed._symmetric_memory as symm

        from . import _pybind

        most = torch.tensor([total_rows], dtype=torch.int64, device=device)
        self.dist.all_reduce(most, op=self.dist.ReduceOp.MAX, group=self.group)
        capacity = max(int(most.item()), 1)             # symmetric allocations have one size on every rank
        buffer = symm.empty((capacity, feat), dtype=dtype, device=device)
        self._handle = symm.rendezvous(buffer, self.group if self.group is not None else self.dist.group.WORLD)
        self._buffer = buffer
        self.compact = buffer[:total_rows]
        self._pulls = []                                # (peer block, wanted rows inside it, unit pointers, halo slice)
        offset = 0
        for peer in range(self.world):
            count = self.want_splits[peer]
            if peer == self.rank or count == 0:
                offset += count if peer != self.rank else 0
                continue
            wanted = (remote[offset:offset + count] - self.bounds[peer]).contiguous()
            block = self._handle.get_buffer(peer, (capacity, feat), dtype)
            unit = torch.arange(count + 1, dtype=wanted.dtype, device=device)
            self._pulls.append((peer, block, wanted, unit, self.own_rows + offset, count))
            offset += count
        self._pulls.sort(key=lambda item: (item[0] - self.rank) % self.world)  # next rank first: no lockstep on one peer
        self._gather_into = _pybind.gather_rows
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        # pulls from different peers run side by side (each is a small launch with its own tail) on a few streams
        self._pull_streams = [torch.cuda.Stream(device) for _ in range(min(4, max(len(self._pulls) - 1, 0)))]

    def _stream_barrier(self) -> None:
        self.dist.all_reduce(self._flag, group=self.group)  # ordered on the current stream; no host wait

    def exchange_rows(self) -> Tuple[int, int]:
        """(rows this rank sends, rows it receives) per step."""
        return int(self.send_rows.numel()), self.halo_rows

    def exchange(self, x_block: torch.Tensor) -> torch.Tensor:
        """Bring the rank's block and its halo together; returns the compact ``[own rows | halo rows]`` matrix."""
        if x_block.data_ptr() != self.own_block.data_ptr():
            self.own_block.copy_(x_block)
        if self.world > 1 and self.transport == "pull":
            self._stream_barrier()
            if not self._pull_streams:
                for _, block, wanted, unit, start, count in self._pulls:
                    self._gather_into(block, wanted, unit, self.compact[start:start + count])
            else:
                main = torch.cuda.current_stream()
                ready = torch.cuda.Event()
                ready.record(main)
                for k, (_, block, wanted, unit, start, count) in enumerate(self._pulls):
                    side = self._pull_streams[k % len(self._pull_streams)]
                    side.wait_event(ready)
                    with torch.cuda.stream(side):
                        self._gather_into(block, wanted, unit, self.compact[start:start + count])
                for side in self._pull_streams:
                    main.wait_stream(side)
            self._stream_barrier()
        elif self.world > 1:
            packed = self.gather_rows(self.own_block, self.send_rows) if self.send_rows.numel() else \
                self.own_block.new_empty((0, self.own_block.size(1)))
            self.dist.all_to_all_single(self.halo, packed, self.want_splits, self.give_splits, group=self.group)
        return self.compact

    def __call__(self, x_block: torch.Tensor) -> torch.Tensor:
        return self.local_spmm(self.rowptr, self.col, self.value, self.exchange(x_block))


class HaloShardedSddmm(HaloShardedSpmm):
    """One rank's share of ``out[e] = <A[row(e)], B[col(e)]>`` over a row-sharded graph.

    The rows of ``A`` an edge needs are the shard's own rows; the rows of ``B`` are its columns, so ``B`` goes through
    the same needed-rows exchange as the dense operand of :class:`HaloShardedSpmm` (same ``bounds``, ``transport``
    and stand-in hooks) and the local SDDMM reads the compact buffer through the relabelled columns.  The result is
    the rank's slice of the edge values, in the order of its CSR slice.
    """

    def __init__(self, rowptr, col, bounds: Sequence[int], feat: int, dtype, device, group=None,
                 local_sddmm: Optional[Callable] = None, gather_rows: Optional[Callable] = None,
                 transport: str = "alltoall", op: str = "dot"):
        super().__init__(rowptr, col, None, bounds, feat, dtype, device, group=group,
                         local_spmm=(lambda *unused: None) if local_sddmm is not None else None,
                         gather_rows=gather_rows, transport=transport)
        if local_sddmm is None:
            from .sddmm_csr import sddmm_csr

            local_sddmm = lambda ptr, c, lhs, rhs: sddmm_csr(ptr, c, lhs, rhs, op, "u", "v")  # noqa: E731
        self.local_sddmm = local_sddmm

    def __call__(self, lhs_block: torch.Tensor, rhs_block: torch.Tensor) -> torch.Tensor:
        return self.local_sddmm(self.rowptr, self.col, lhs_block, self.exchange(rhs_block))



class ShardedGatLayer:
    """A GAT-style attention layer over a row-sharded graph.

    Per head ``h``: ``logit[e, h] = left[row(e), h] + right[col(e), h]``, LeakyReLU, softmax over the edges of each
    destination row, ``out[r, h, :] = sum_e alpha[e, h] * x[col(e), h, :]``.  Rows are the shard's own, so the
    softmax needs no exchange; ``right`` (``[rows, heads]``) and ``x`` (``[rows, heads, width]``) go through the
    needed-rows exchange, ``left`` is local.

    ``fused=False`` composes the layer from the sharded operators (sharded SDDMM ``add``, ``scatter_softmax``, fused
    per-head aggregation).  ``fused=True`` exchanges ``right`` and ``x`` into their compact buffers and runs the local
    layer as :func:`ops_gnn.gat_aggregate` (two launches, no ``[E, H]`` softmax tensor).
    """

    def __init__(self, rowptr, col, bounds: Sequence[int], heads: int, width: int, dtype, device, group=None,
                 transport: str = "alltoall", negative_slope: float = 0.2, fused: bool = False):
        from .bspmm import bspmm
        from .ptr2ind import ptr2ind
        from .scatter_softmax import scatter_softmax

        self.heads, self.width, self.slope, self.fused = heads, width, negative_slope, fused
        self.rows = rowptr.numel() - 1
        self.rowptr = rowptr
        self.edge_rows = ptr2ind(rowptr, col.numel())
        if fused:
            self.features = HaloShardedSpmm(rowptr, col, None, bounds, heads * width, dtype, device, group=group,
                                            transport=transport, local_spmm=lambda *unused: None)
            self.halves = HaloShardedSpmm(rowptr, col, None, bounds, heads, dtype, device, group=group,
                                          transport=transport, local_spmm=lambda *unused: None)
            return
        self.softmax = scatter_softmax
        self.logits = HaloShardedSddmm(rowptr, col, bounds, heads, dtype, device, group=group, transport=transport, op="add")
        self.aggregate = HaloShardedSpmm(
            rowptr, col, None, bounds, heads * width, dtype, device, group=group, transport=transport,
            local_spmm=lambda ptr, c, alpha, x: bspmm(ptr, c, x.view(-1, heads, width), "mul", "sum", rhs=alpha))

    def __call__(self, x_block: torch.Tensor, left_block: torch.Tensor, right_block: torch.Tensor) -> torch.Tensor:
        if self.fused:
            from .gat_aggregate import gat_aggregate

            x_all = self.features.exchange(x_block.reshape(self.rows, self.heads * self.width))
            right_all = self.halves.exchange(right_block)
            out = gat_aggregate(self.rowptr, self.features.col, x_all.view(-1, self.heads, self.width), left_block, right_all,
                                self.slope, edge_rows=self.edge_rows)
            return out.view(self.rows, self.heads * self.width)
        scores = torch.nn.functional.leaky_relu(self.logits(left_block, right_block), self.slope)
        self.aggregate.value = self.softmax(scores, self.edge_rows, 0, self.rows).unsqueeze(-1)
        return self.aggregate(x_block.reshape(self.rows, self.heads * self.width))


def staged_row_bounds(rowptr: torch.Tensor, fractions: Sequence[float], row_cost: float = 4.0) -> List[int]:
    """Row boundaries that cut a shard into ``len(fractions)`` consecutive stages holding these shares of its work
    (edges + ``row_cost`` per row)."""
    rows = rowptr.numel() - 1
    total = float(sum(fractions))
    if rows < 0 or total <= 0 or any(f < 0 for f in fractions):
        raise ValueError("stage fractions must be non-negative and not all zero")
    work = rowptr.to(torch.float64) - float(rowptr[0]) + row_cost * torch.arange(rows + 1, dtype=torch.float64,
                                                                              device=rowptr.device)
    done, bounds = 0.0, [0]
    for f in list(fractions)[:-1]:
        done += f / total
        target = torch.tensor([done * float(work[-1])], dtype=torch.float64, device=rowptr.device)
        bounds.append(min(max(int(torch.searchsorted(work, target)), bounds[-1]), rows))
    bounds.append(rows)
    return bounds


class StagedHaloSpmm:
    """Needed-rows sharded SpMM whose exchange and product overlap stage by stage.

    :class:`HaloShardedSpmm` finishes its whole exchange before the local SpMM starts.  Here the rank's rows are cut
    into consecutive stages (``stage_fractions`` of the shard's work).  Stage ``k`` needs the rows of ``X`` its
    columns reference that no earlier stage has already brought in; the compact buffer is laid out as
    ``[own rows | new rows of stage 1 grouped by owner | new rows of stage 2 ... ]``.  The exchanges of all stages run
    back to back on a side stream; the product of stage ``k`` waits only for exchange ``k`` and writes its own row
    range of the output, so while stage ``k`` computes, stage ``k + 1`` is on the wire.  Every output row is still
    produced by one kernel over all of its edges, in the order of the one-GPU product.

    ``transport="alltoall"``: per stage, pack the wanted rows per peer (the CSR engine run as a gather) and one NCCL
    all-to-all with uneven splits.  ``transport="push"`` (CUDA only): the compact buffers live in symmetric memory and
    the gather kernel writes each wanted row straight into the requesting peer's buffer with plain peer stores - the
    pack IS the transfer, no send buffer and no NCCL data path; stream-ordered one-element all-reduces mark "every
    peer's stage-k rows have landed" and, at the start of a step, "nobody still reads last step's buffers".
    ``transport="copy"`` (CUDA only): the same symmetric buffers, but the rows are packed into a local send buffer per
    stage and moved with one ``cudaMemcpyAsync`` per peer and stage (``_pybind.copy_rows_async``), which the driver
    runs on the copy engines: the transfer takes no SM slot and no issue bandwidth from the product running beside it
    (NCCL's all-to-all kernels and the pushing gather kernel both slowed down, and slowed the product, when they
    overlapped it).  The same one-element all-reduces act as barriers; pass ``barrier_group`` (a
    :func:`high_priority_group`) so that they are not queued behind the product's thread blocks.

    The exchange kernel is the bounded row gather (``_pybind.gather_rows_into``): one launch per stage serves every
    peer, and its grid is capped at ``exchange_ctas`` thread blocks, because it runs beside a product and is bound by
    NVLink latency, not by the SMs (one block per SM moves what the link takes and leaves room for the product's blocks).

    ``spmm_into(ptr, col, value, x, out)`` and ``gather_rows(x, index, outs, max_ctas)`` default to the CUDA kernels;
    the CPU tests pass stand-ins.
    """

    def __init__(self, rowptr, col, value, bounds: Sequence[int], feat: int, dtype, device, group=None,
                 stage_fractions: Sequence[float] = (0.25, 0.25, 0.25, 0.25), row_cost: float = 4.0,
                 transport: str = "alltoall", spmm_into: Optional[Callable] = None,
                 gather_rows: Optional[Callable] = None, exchange_ctas: int = 148, barrier_group=None,
                 copy_streams: int = 4):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.barrier_group = barrier_group if barrier_group is not None else group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if len(bounds) != self.world + 1:
            raise ValueError("bounds must hold one row range per rank")
        if transport not in ("alltoall", "push", "copy"):
            raise ValueError("transport must be 'alltoall', 'push' or 'copy'")
        self.transport, self.feat, self.dtype, self.device = transport, feat, dtype, device
        self.exchange_ctas = int(exchange_ctas)
        self.bounds = [int(b) for b in bounds]
        self.own_first, own_last = self.bounds[self.rank], self.bounds[self.rank + 1]
        self.own_rows = own_last - self.own_first
        self.stage_rows = staged_row_bounds(rowptr, stage_fractions, row_cost)
        stages = len(self.stage_rows) - 1
        edges = torch.tensor(self.bounds, dtype=col.dtype, device=device)
        cut = [int(v) for v in rowptr[torch.tensor(self.stage_rows, device=rowptr.device)].tolist()]

        # per stage: the remote rows no earlier stage brings in, what every peer wants of this rank, and the splits
        seen = col.new_empty(0)
        fresh, self.want_splits, self.give_splits, self.send_rows = [], [], [], []
        for k in range(stages):
            needed = torch.unique(col[cut[k]:cut[k + 1]])
            remote = needed[(needed < self.own_first) | (needed >= own_last)]
            new = remote[~torch.isin(remote, seen)] if seen.numel() else remote      # sorted: grouped by owner
            seen = torch.sort(torch.cat([seen, new])).values
            owner = torch.searchsorted(edges, new, right=True) - 1
            want = torch.bincount(owner, minlength=self.world)
            give = torch.empty_like(want)
            dist.all_to_all_single(give, want, group=group)
            want_list, give_list = [int(c) for c in want.tolist()], [int(c) for c in give.tolist()]
            wanted_of_me = torch.empty(sum(give_list), dtype=col.dtype, device=device)
            dist.all_to_all_single(wanted_of_me, new.contiguous(), give_list, want_list, group=group)
            rows_out = (wanted_of_me - self.own_first).contiguous()
            if rows_out.numel() and (int(rows_out.min()) < 0 or int(rows_out.max()) >= self.own_rows):
                raise RuntimeError("a peer asked for rows outside this rank's block: shard bounds disagree between ranks")
            fresh.append(new)
            self.want_splits.append(want_list)
            self.give_splits.append(give_list)
            self.send_rows.append(rows_out)
        self.halo_counts = [int(n.numel()) for n in fresh]
        self.halo_rows = sum(self.halo_counts)
        self.halo_start = [self.own_rows]
        for count in self.halo_counts:
            self.halo_start.append(self.halo_start[-1] + count)

        # compact column ids: own rows first, then the halo in the order it is received
        arrival = torch.cat(fresh) if stages else col.new_empty(0)
        ids, order = torch.sort(arrival)
        is_own = (col >= self.own_first) & (col < own_last)
        if ids.numel():
            at = torch.searchsorted(ids, col).clamp_(max=ids.numel() - 1)
            compact = torch.where(is_own, col - self.own_first, self.own_rows + order[at])
        else:
            compact = col - self.own_first
        self.col = compact.contiguous()
        self.stage_ptr = [(rowptr[self.stage_rows[k]:self.stage_rows[k + 1] + 1] - cut[k]).contiguous()
                          for k in range(stages)]
        self.stage_col = [self.col[cut[k]:cut[k + 1]] for k in range(stages)]
        self.stage_val = [None if value is None else value[cut[k]:cut[k + 1]] for k in range(stages)]

        total_rows = self.own_rows + self.halo_rows
        if transport in ("push", "copy"):
            self._setup_push(total_rows)
        else:
            self.compact = torch.empty((total_rows, feat), dtype=dtype, device=device)
        self.own_block = self.compact[:self.own_rows]
        if spmm_into is None or gather_rows is None:
            from . import _pybind

            spmm_into = spmm_into or _pybind.csr_spmm_into
            gather_rows = gather_rows or _pybind.gather_rows_into
        self.spmm_into, self.gather_rows = spmm_into, gather_rows
        on_gpu = device.type == "cuda"
        # High priority: when a pack (or push) kernel and a product are both pending, free SM slots go to the exchange
        # first, so the next stage's rows get on the wire while the current product computes.  Without it the small
        # exchange kernels queue behind the product's thread blocks and the stages run one after the other (measured).
        self.comm_stream = torch.cuda.Stream(device, priority=-1) if on_gpu else None
        # The all-to-all transport packs on a stream of its own, into one send buffer per stage, so the pack of stage
        # k + 1 runs beside the all-to-all of stage k instead of behind it (measured at eight GPUs with one stream:
        # 4 x (0.9 ms pack + 2.2 ms all-to-all) in a row).
        self.pack_stream = torch.cuda.Stream(device, priority=-1) if (on_gpu and transport != "push") else None
        self._packed = [torch.empty((int(rows.numel()), feat), dtype=dtype, device=device) for rows in self.send_rows] \
            if transport != "push" else []
        self.copy_streams = [torch.cuda.Stream(device, priority=-1) for _ in range(max(1, int(copy_streams)))] \
            if (on_gpu and transport == "copy") else []
        if transport == "copy":
            from . import _pybind

            self._copy_rows = _pybind.copy_rows_async
        self.timing = False       # set it to collect CUDA events per phase of the next step (see phase_ms)
        self._events = None

    # ---- push transport: symmetric memory and where each peer wants this rank's rows ------------------------------
    def _setup_push(self, total_rows: int) -> None:
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only, no multicast binding
        import torch.distributed._symmetric_memory as symm

        dist, device = self.dist, self.device
        most = torch.tensor([total_rows], dtype=torch.int64, device=device)
        dist.all_reduce(most, op=dist.ReduceOp.MAX, group=self.group)
        capacity = max(int(most.item()), 1)             # symmetric allocations have one size on every rank
        buffer = symm.empty((capacity, self.feat), dtype=self.dtype, device=device)
        self._handle = symm.rendezvous(buffer, self.group if self.group is not None else dist.group.WORLD)
        self._buffer = buffer
        self.compact = buffer[:total_rows]
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        # For every stage, tell each owner where in this rank's compact buffer its rows go; learn the same from the peers.
        self._push = []           # per stage: where each peer wants this rank's rows, in the order of send_rows[k]
        for k, want in enumerate(self.want_splits):
            starts, at = [], self.halo_start[k]
            for count in want:
                starts.append(at)
                at += count
            mine = torch.tensor(starts, dtype=torch.int64, device=device)
            theirs = torch.empty_like(mine)
            dist.all_to_all_single(theirs, mine, group=self.group)
            theirs = [int(v) for v in theirs.tolist()]
            targets = []
            for peer, count in enumerate(self.give_splits[k]):
                if count:                           # nobody asks itself, so the segments are exactly the peers' shares
                    block = self._handle.get_buffer(peer, (capacity, self.feat), self.dtype)
                    targets.append(block[theirs[peer]:theirs[peer] + count])
            self._push.append(targets)              # in the order of send_rows[k]: consecutive slices of a packed stage

    def _stream_barrier(self) -> None:
        self.dist.all_reduce(self._flag, group=self.barrier_group)  # ordered on the current stream; no host wait

    def exchange_rows(self) -> Tuple[int, int]:
        """(rows this rank sends, rows it receives) per step, over all stages."""
        return sum(int(r.numel()) for r in self.send_rows), self.halo_rows

    def _mark(self, name: str) -> None:
        if self._events is not None:
            event = torch.cuda.Event(enable_timing=True)
            event.record(torch.cuda.current_stream())
            self._events.append((name, event))

    def _exchange_stage(self, k: int) -> None:
        halo = self.compact[self.halo_start[k]:self.halo_start[k + 1]]
        if self.transport == "push":
            if self._push[k]:                       # one launch stores into every peer's buffer: all of them receive at once
                self.gather_rows(self.own_block, self.send_rows[k], self._push[k], self.exchange_ctas)
            self._mark(f"pack{k}")
            self._stream_barrier()                  # every peer's stage-k rows have landed here too
        elif self.transport == "copy":
            self._stream_barrier()                  # the copies of stage k were joined into this stream by the caller
        else:
            if self.pack_stream is None:
                self._pack_stage(k)
            self.dist.all_to_all_single(halo, self._packed[k], self.want_splits[k], self.give_splits[k], group=self.group)
        self._mark(f"exchange{k}")

    def _pack_stage(self, k: int) -> None:
        if self._packed[k].size(0):     # a local gather, bound by HBM: the kernel's own grid (0), not the NVLink-sized cap
            self.gather_rows(self.own_block, self.send_rows[k], [self._packed[k]], 0)
        self._mark(f"pack{k}")

    def __call__(self, x_block: torch.Tensor) -> torch.Tensor:
        if x_block.data_ptr() != self.own_block.data_ptr():
            self.own_block.copy_(x_block)
        stages = len(self.stage_ptr)
        out = self.own_block.new_empty((self.own_rows, self.feat))
        self._events = [] if (self.timing and self.comm_stream is not None) else None
        if self.comm_stream is None:                # CPU ranks (tests): the same order without streams
            for k in range(stages):
                if self.world > 1:
                    self._exchange_stage(k)
            for k in range(stages):
                first, last = self.stage_rows[k], self.stage_rows[k + 1]
                self.spmm_into(self.stage_ptr[k], self.stage_col[k], self.stage_val[k], self.compact, out[first:last])
            return out
        main, comm, pack = torch.cuda.current_stream(), self.comm_stream, self.pack_stream
        comm.wait_stream(main)                      # the block is in place; last step's products are enqueued before
        landed, packed = [], []
        with torch.cuda.stream(comm):
            self._mark("start")
        if pack is not None and self.world > 1:
            pack.wait_stream(main)                  # main has waited for last step's exchanges: the send buffers are free
            with torch.cuda.stream(pack):
                for k in range(stages):
                    self._pack_stage(k)
                    event = torch.cuda.Event()
                    event.record(pack)
                    packed.append(event)
        with torch.cuda.stream(comm):
            if self.world > 1 and self.transport in ("push", "copy"):
                self._stream_barrier()              # nobody still reads the halo this step overwrites
            free = torch.cuda.Event()
            free.record(comm)
            for k in range(stages):
                if self.world > 1:
                    if self.transport == "copy":
                        self._copy_stage(k, packed[k], free, comm)
                    elif packed:
                        comm.wait_event(packed[k])
                    self._exchange_stage(k)
                event = torch.cuda.Event()
                event.record(comm)
                landed.append(event)
        for k in range(stages):
            main.wait_event(landed[k])
            first, last = self.stage_rows[k], self.stage_rows[k + 1]
            self.spmm_into(self.stage_ptr[k], self.stage_col[k], self.stage_val[k], self.compact, out[first:last])
            self._mark(f"product{k}")
        comm.wait_stream(main)                      # scratch allocated on either stream is not reused across the join
        return out

    def _copy_stage(self, k: int, packed_ready, halo_free, comm) -> None:
        """One copy-engine transfer per peer from the packed rows of stage ``k`` into the peers' buffers, spread over
        the copy streams; ``comm`` then waits for all of them."""
        at = 0
        for n, target in enumerate(self._push[k]):
            stream = self.copy_streams[n % len(self.copy_streams)]
            stream.wait_event(packed_ready)
            stream.wait_event(halo_free)
            with torch.cuda.stream(stream):
                self._copy_rows(self._packed[k][at:at + target.size(0)], target)
                done = torch.cuda.Event()
                done.record(stream)
            comm.wait_event(done)
            at += target.size(0)

    def phase_ms(self):
        """After a step run with ``timing = True`` (and a device synchronise): milliseconds from the step's start to the
        end of every phase, in the order the phases were enqueued."""
        if not self._events:
            return {}
        start = self._events[0][1]
        return {name: start.elapsed_time(event) for name, event in self._events[1:]}
