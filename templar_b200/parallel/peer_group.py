"""Nodes that share a box exchange their gradients through peer memory instead of the object store.

When several nodes (uids) run as the ranks of one process group on one 8-GPU machine, each of them compresses its
pseudo-gradient into buffers of the symmetric heap.  A peer on the same box then needs no upload, download,
deserialisation or host-to-device copy to use that payload: its aggregation kernel reads the packed indices and
values straight from the owner's memory over NVLink (``WindowEngine.outer_step(peers=[("rank", r), ...])``).
Uploads to the object store still happen, for the peers and validators elsewhere.

:class:`LocalPeerGroup` is the small amount of bookkeeping this needs: which uid runs on which rank, and a board on
which every rank posts the window its buffers currently hold, so that a payload left over from an earlier window is
never taken for the current one.  On CPU (gloo) there is no peer memory; the payloads are exchanged with an
all-gather, which keeps the protocol testable without GPUs.

The reference has no counterpart: every gradient travels through its bucket, also between miners of one machine
(src/tplr/comms.py:1287-1378, :1631-2117).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native


class LocalPeerGroup:
    def __init__(self, uid: int, *, rank: int, world_size: int, heap=None, group=None, device=None):
        self.uid, self.rank, self.world_size, self.heap, self.group = int(uid), rank, world_size, heap, group
        self.device = torch.device(device) if device is not None else (heap.device if heap is not None else torch.device("cpu"))
        uids = [None] * world_size
        if world_size > 1:
            dist.all_gather_object(uids, int(uid), group=group)
        else:
            uids = [int(uid)]
        if len(set(uids)) != len(uids):
            raise ValueError(f"co-located nodes need distinct uids, got {uids}")
        self.uids: list[int] = uids
        self.rank_of = {u: r for r, u in enumerate(uids)}
        # board[r] = window whose payload rank r's buffers hold (-1: none); every rank keeps a full copy
        if heap is not None:
            self.board = heap.alloc(max(world_size, 2), torch.int64)
        else:
            self.board = torch.zeros(max(world_size, 2), dtype=torch.int64, device=self.device)
        self.board.fill_(-1)
        self._engine = None
        self.barrier()

    # -- wiring ---------------------------------------------------------------------------------
    def attach(self, engine) -> None:
        """``engine``: this rank's window engine (one node per rank: ``world_size`` 1, buffers on the shared heap)."""
        if engine.world_size != 1:
            raise ValueError("co-located nodes are whole nodes: their engines are not sharded over the ranks")
        self._engine = engine
        engine.peer_group = self

    def barrier(self) -> None:
        if self.world_size == 1:
            return
        if self.heap is not None:
            self.heap.barrier()
        else:
            dist.barrier(group=self.group)

    # -- per window -----------------------------------------------------------------------------
    def publish(self, window: int) -> None:
        """This rank's payload buffers now hold ``window``'s gradient: post it on every rank's board.  Stream
        ordered after the compress kernels; :meth:`exchange` makes it visible."""
        if self.heap is not None and self.world_size > 1:
            for r in range(self.world_size):
                native.check(native.lib().tplr_store_i64(self.heap.peer_ptr(self.board, r) + 8 * self.rank, int(window),
                                                         native.stream_ptr()), "store_i64")
        else:
            self.board[self.rank] = int(window)

    def exchange(self) -> None:
        """All payloads of this window are in place and the boards agree (a barrier; on CPU also the all-gather that
        stands in for peer memory)."""
        if self.world_size == 1:
            return
        if self.heap is None:
            cells = [torch.zeros(1, dtype=torch.int64) for _ in range(self.world_size)]
            dist.all_gather(cells, self.board[self.rank: self.rank + 1].cpu(), group=self.group)
            self.board[: self.world_size] = torch.cat(cells).to(self.board.device)
            eng = self._engine
            if eng is not None:
                idx = [torch.empty_like(eng.own_idx) for _ in range(self.world_size)]
                val = [torch.empty_like(eng.own_val) for _ in range(self.world_size)]
                dist.all_gather(idx, eng.own_idx, group=self.group)
                dist.all_gather(val, eng.own_val, group=self.group)
                eng.rank_payloads = {r: (idx[r], val[r]) for r in range(self.world_size)}
        self.barrier()

    def fresh(self, window: int) -> dict[int, int]:
        """{uid: rank} of the co-located nodes whose buffers hold ``window``'s payload (host read of the board)."""
        board = self.board[: self.world_size].cpu().tolist()
        return {u: r for r, u in enumerate(self.uids) if board[r] == int(window)}
