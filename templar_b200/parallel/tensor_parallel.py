"""Tensor parallelism with sequence-sharded activations on fused compute+collective kernels.

Plan (the reference's, torchtitan models/llama3/infra/parallelize.py:151-219): q/k/v and w1/w3 are
split by output feature (column parallel), wo and w2 by input feature (row parallel), and the
activations between blocks are sharded by token.  Where the reference runs an NCCL all-gather
before a cuBLAS GEMM and a cuBLAS GEMM before an NCCL reduce-scatter, this module issues ONE
kernel for each pair (``tplr_gemm2_gather`` / ``tplr_gemm2_scatter``): the collective moves over
NVLink peer memory inside the GEMM launch, tile by tile.

Buffers live on the symmetric heap: two gather buffers (alternated so that a rank may refill one
while a slower peer still copies the other) and one buffer for the rows a rank owns of a
reduce-scattered product, into which all ranks' GEMM epilogues reduce-add their partial tiles.
Every fused call is preceded by one stream-ordered heap barrier, which both publishes the caller's
rows to its peers and proves that all peers are done with the buffers of the call before the
previous one; the reduce-scatter is followed by a second one, after which the sums are complete.
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import functional as OF
from ..ops import native
from .symmetric import SymmetricHeap

_MAX_CHUNKS = 1024


class TensorParallel:
    """Workspace and launcher of the fused kernels for one tensor-parallel group.

    ``rows`` is the number of tokens of the full (gathered) activation, ``width`` the widest
    activation that is gathered or reduce-scattered (the model dimension)."""

    def __init__(self, heap: SymmetricHeap, rows: int, width: int, n_comm_pairs: int | None = None,
                 reduce_dtype: torch.dtype = torch.bfloat16):
        self.heap, self.rank, self.world = heap, heap.rank, heap.world_size
        native.require(rows % (128 * self.world) == 0, "tensor parallel: rows must be a multiple of 128 * world")
        native.require(rows // 128 <= _MAX_CHUNKS, "tensor parallel: too many rows")
        self.rows, self.width = rows, width
        self.rows_per_rank = rows // self.world
        self.n_comm_pairs = n_comm_pairs
        self.device = heap.device
        self._g = [heap.alloc(rows * width, torch.bfloat16) for _ in range(2)]
        # reduce-scatter target: bf16 sums like NCCL's bf16 reduce-scatter, or fp32 sums at twice the NVLink bytes
        self.reduce_dtype = reduce_dtype
        self._r = heap.alloc(self.rows_per_rank * width, reduce_dtype)
        self._gflags = [torch.zeros(_MAX_CHUNKS, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._g_next = 0
        self._epoch = 0
        torch.cuda.synchronize(self.device)
        heap.barrier()

    # -- buffers --------------------------------------------------------------------------------
    def gather_buffer(self, width: int) -> tuple[int, torch.Tensor, torch.Tensor]:
        """Next gather buffer: (slot, full [rows, width] view, this rank's [rows/world, width] rows)."""
        native.require(width <= self.width, "tensor parallel: activation wider than the workspace")
        slot = self._g_next
        self._g_next ^= 1
        full = self._g[slot][: self.rows * width].view(self.rows, width)
        own = full[self.rank * self.rows_per_rank:(self.rank + 1) * self.rows_per_rank]
        return slot, full, own

    def _next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    def _comm_pairs(self, flops: float, link_bytes: float, tiles: int) -> int:
        """CTA pairs set aside for the gather.  The tiles of the local shard need no peer data, so the
        peers' rows have to arrive within the remaining (world-1)/world of the GEMM's time; one copier
        CTA sustains about 45 GB/s (160 KB of loads in flight over NVLink), and more than 16 of them
        only saturate the link."""
        if self.n_comm_pairs is not None:
            return self.n_comm_pairs
        if self.world == 1:
            return 1
        t_remote = flops / 1.4e15 * (self.world - 1) / self.world
        need_gbs = min(link_bytes / max(t_remote, 1e-6) / 1e9, 720.0)
        pairs = max(1, min(8, -(-int(need_gbs / 45.0 + 0.999) // 2)))
        if tiles <= 2 * 74:
            # a GEMM of at most two waves leaves CTA pairs idle anyway: spend them on the gather
            pairs = max(pairs, min(12, 74 - -(-tiles // 2)))
        return pairs

    # -- fused kernels ----------------------------------------------------------------------------
    def ag_gemm(self, slot: int, width: int, other: torch.Tensor, *, gathered: str = "A", a_mn: bool = False,
                b_mn: bool = False, out: torch.Tensor | None = None, accumulate: bool = False,
                out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """GEMM whose operand ``gathered`` is gather buffer ``slot`` ([rows, width], token-sharded over ranks).

        gathered == "A": ``C = G other^T`` (``a_mn`` False: G is [M, K]; True: G is [K, M] and K is the token axis).
        gathered == "B": ``C = op(other) G`` with ``b_mn`` True (G is [K, N], K the token axis)."""
        full = self._g[slot][: self.rows * width].view(self.rows, width)
        if gathered == "A":
            a, b = full, other
        else:
            a, b = other, full
        M = a.shape[1] if a_mn else a.shape[0]
        K = a.shape[0] if a_mn else a.shape[1]
        N = b.shape[1] if b_mn else b.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=self.device)
            accumulate = False
        epi = 0 if out.dtype == torch.bfloat16 else (1 if accumulate else 2)
        self.heap.barrier()
        bases = [self.heap.peer_ptr(self._g[slot], r) for r in range(self.world)]
        err = native.lib().tplr_gemm2_gather(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            int(a_mn), int(b_mn), epi, 1 if gathered == "A" else 2, self.world, self.rank, self.rows_per_rank,
            native.ptr_array(bases), self._gflags[slot].data_ptr(), ctypes.c_uint(self._next_epoch()),
            self._comm_pairs(2.0 * M * N * K, (self.world - 1) * self.rows_per_rank * width * 2,
                             -(-M // 256) * -(-N // 256)),
            OF.status_word(self.device).data_ptr(), native.stream_ptr())
        native.check(err, "tplr_gemm2_gather")
        return out

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, *, b_mn: bool = False,
                out: torch.Tensor | None = None) -> torch.Tensor:
        """``out = reduce_scatter_rows(a op(b))``: a is [rows, K_local]; returns this rank's [rows/world, N] rows."""
        M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        native.require(M == self.rows and N <= self.width, "gemm_rs: shape outside the workspace")
        ws = self._r[: self.rows_per_rank * N].view(self.rows_per_rank, N)
        ws.zero_()
        self.heap.barrier()
        outs = [self.heap.peer_ptr(self._r, r) for r in range(self.world)]
        err = native.lib().tplr_gemm2_scatter(
            a.data_ptr(), b.data_ptr(), M, N, K, a.stride(0), b.stride(0), 0, int(b_mn), self.world, self.rank,
            self.rows_per_rank, native.ptr_array(outs), N, int(self.reduce_dtype == torch.float32),
            OF.status_word(self.device).data_ptr(), native.stream_ptr())
        native.check(err, "tplr_gemm2_scatter")
        self.heap.barrier()
        if out is None:
            return ws.to(torch.bfloat16, copy=True)
        out.copy_(ws)
        return out

    def check(self) -> None:
        """Host sync; raises if a bounded wait expired in a fused kernel or a barrier."""
        self.heap.check()
        st = OF.status_word(self.device)
        v = int(st.item())
        if v:
            st.zero_()
            raise TimeoutError(f"tensor-parallel kernel gave up waiting for a peer (status {v:#x})")


class GatheredWeight:
    """A weight [N, K] whose rows are sharded over the ranks (the FSDP layout) and whose all-gather is fused
    into the first GEMM that consumes it: ``linear(x)`` returns ``x W^T`` while copier CTAs of the same
    launch pull the peers' row shards into this rank's full-size buffer, tile columns of the local shard
    first.  After the call the buffer holds the whole weight, so the backward GEMMs of the same layer need
    no communication.  Replaces FSDP2's per-block all-gather + cuBLAS (the reference's
    torchtitan models/llama3/infra/parallelize.py:325-375 applied by src/tplr/model_factory.py:286-331)."""

    def __init__(self, heap: SymmetricHeap, n_rows: int, k: int, n_comm_pairs: int | None = None):
        self.heap, self.rank, self.world = heap, heap.rank, heap.world_size
        native.require(n_rows % (128 * self.world) == 0, "gathered weight: rows must be a multiple of 128 * world")
        native.require(n_rows // 128 <= _MAX_CHUNKS and k % 8 == 0, "gathered weight: shape not supported")
        self.n_rows, self.k, self.rows_per_rank = n_rows, k, n_rows // self.world
        self.device = heap.device
        self.n_comm_pairs = n_comm_pairs
        self._full = heap.alloc(n_rows * k, torch.bfloat16)
        self.full = self._full.view(n_rows, k)
        self.own = self.full[self.rank * self.rows_per_rank:(self.rank + 1) * self.rows_per_rank]
        self._flags = torch.zeros(_MAX_CHUNKS, dtype=torch.int32, device=self.device)
        self._epoch = 0

    def linear(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``y[M, N] = x[M, K] W^T`` with the gather of W inside the launch (x: bf16, rows contiguous)."""
        M, K = x.shape
        native.require(K == self.k, "gathered weight: inner dimensions differ")
        if out is None:
            out = torch.empty(M, self.n_rows, dtype=torch.bfloat16, device=self.device)
        self._epoch += 1
        link = (self.world - 1) * self.rows_per_rank * K * 2
        pairs = self.n_comm_pairs
        if pairs is None:
            t_remote = 2.0 * M * self.n_rows * K / 1.4e15 * (self.world - 1) / max(self.world, 1)
            pairs = max(1, min(8, -(-int(min(link / max(t_remote, 1e-6) / 1e9, 720.0) / 45.0 + 0.999) // 2)))
        self.heap.barrier()
        bases = [self.heap.peer_ptr(self._full, r) for r in range(self.world)]
        err = native.lib().tplr_gemm2_gather(
            x.data_ptr(), self.full.data_ptr(), out.data_ptr(), M, self.n_rows, K, x.stride(0), K, out.stride(0),
            0, 0, 0, 2, self.world, self.rank, self.rows_per_rank, native.ptr_array(bases), self._flags.data_ptr(),
            ctypes.c_uint(self._epoch), pairs, OF.status_word(self.device).data_ptr(), native.stream_ptr())
        native.check(err, "tplr_gemm2_gather")
        return out


def reduce_scatter_rows(part: torch.Tensor, rank: int, world: int, group=None) -> torch.Tensor:
    """Sum ``part`` [rows, n] over ranks and return this rank's block of rows/world rows (NCCL: one
    reduce-scatter; other backends: all-reduce and slice)."""
    import torch.distributed as dist

    n = part.shape[0] // world
    if dist.get_backend(group) == "nccl":
        out = torch.empty(n, part.shape[1], dtype=part.dtype, device=part.device)
        dist.reduce_scatter_tensor(out, part.contiguous(), group=group)
        return out
    full = part.clone()
    dist.all_reduce(full, group=group)
    return full[rank * n:(rank + 1) * n].clone()


def all_gather_rows(shard: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Concatenation over ranks of ``shard`` [rows/world, n] along the rows."""
    import torch.distributed as dist

    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return torch.cat(parts, dim=0)


class CollectiveTensorParallel:
    """Same interface as :class:`TensorParallel` on ``torch.distributed`` collectives and plain matmuls
    (any backend, any dtype).  It is the CPU/gloo stand-in for tests of the sharding logic and the
    library baseline that the fused kernels are compared with."""

    def __init__(self, rows: int, width: int, rank: int, world: int, group=None, device="cpu",
                 dtype: torch.dtype = torch.float32):
        self.rows, self.width, self.rank, self.world, self.group = rows, width, rank, world, group
        self.rows_per_rank = rows // world
        self.device = torch.device(device)
        self._g = [torch.zeros(rows * width, dtype=dtype, device=self.device) for _ in range(2)]
        self._g_next = 0

    def gather_buffer(self, width: int):
        slot = self._g_next
        self._g_next ^= 1
        full = self._g[slot][: self.rows * width].view(self.rows, width)
        return slot, full, full[self.rank * self.rows_per_rank:(self.rank + 1) * self.rows_per_rank]

    def ag_gemm(self, slot, width, other, *, gathered="A", a_mn=False, b_mn=False, out=None, accumulate=False,
                out_dtype=None):
        full = self._g[slot][: self.rows * width].view(self.rows, width)
        own = full[self.rank * self.rows_per_rank:(self.rank + 1) * self.rows_per_rank].clone()
        full.copy_(all_gather_rows(own, self.world, self.group))
        a, b = (full, other) if gathered == "A" else (other, full)
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        c = A.float() @ Bt.float()
        if out is None:
            return c.to(out_dtype or a.dtype)
        if accumulate:
            out.add_(c.to(out.dtype))
        else:
            out.copy_(c)
        return out

    def gemm_rs(self, a, b, *, b_mn=False, out=None):
        part = (a.float() @ (b.float() if b_mn else b.float().t())).to(a.dtype)
        res = reduce_scatter_rows(part, self.rank, self.world, self.group)
        if out is None:
            return res
        out.copy_(res)
        return out

    def check(self) -> None:
        return None


# --------------------------------------------------------------------------------------------- #
# autograd pairs
# --------------------------------------------------------------------------------------------- #
class _ColumnParallel(torch.autograd.Function):
    """y[T, N/w] = all_gather(x)[T, K] W^T; backward reduce-scatters dx and re-gathers x for dW."""

    @staticmethod
    def forward(ctx, x_shard, w, tp: TensorParallel, main_grad):
        K = x_shard.shape[-1]
        slot, _, own = tp.gather_buffer(K)
        own.copy_(x_shard.reshape(-1, K))
        y = tp.ag_gemm(slot, K, w)
        ctx.save_for_backward(x_shard, w)
        ctx.tp, ctx.main_grad = tp, main_grad
        return y

    @staticmethod
    def backward(ctx, dy):
        x_shard, w = ctx.saved_tensors
        tp: TensorParallel = ctx.tp
        K = x_shard.shape[-1]
        dy = dy.contiguous()
        dw = None
        if ctx.needs_input_grad[1] or ctx.main_grad is not None:
            slot, _, own = tp.gather_buffer(K)
            own.copy_(x_shard.reshape(-1, K))
            if ctx.main_grad is not None:      # dW += dy^T X, accumulated in fp32 by the GEMM epilogue
                tp.ag_gemm(slot, K, dy, gathered="B", a_mn=True, b_mn=True, out=ctx.main_grad, accumulate=True)
            else:
                dw = tp.ag_gemm(slot, K, dy, gathered="B", a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = tp.gemm_rs(dy, w, b_mn=True).view_as(x_shard)
        return dx, dw, None, None


class _RowParallel(torch.autograd.Function):
    """y[T/w, N] = reduce_scatter(x[T, K/w] W^T); backward gathers dy once for dx and dW."""

    @staticmethod
    def forward(ctx, x, w, tp: TensorParallel, main_grad):
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.main_grad = tp, main_grad
        return tp.gemm_rs(x.reshape(-1, x.shape[-1]), w)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        tp: TensorParallel = ctx.tp
        N = dy_shard.shape[-1]
        slot, full, own = tp.gather_buffer(N)
        own.copy_(dy_shard.reshape(-1, N))
        # dx = all_gather(dy) W : the gather lands dy in `full`, which the weight gradient then reads locally
        dx = tp.ag_gemm(slot, N, w, b_mn=True).view_as(x)
        dw = None
        x2 = x.reshape(-1, x.shape[-1])
        if ctx.main_grad is not None:
            OF.gemm(full, x2, a_mn=True, b_mn=True, out=ctx.main_grad, accumulate=True)
        elif ctx.needs_input_grad[1]:
            dw = OF.gemm(full, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
        return dx, dw, None, None


def column_parallel_linear(x_shard: torch.Tensor, w_local: torch.Tensor, tp: TensorParallel,
                           main_grad: torch.Tensor | None = None) -> torch.Tensor:
    """``x_shard`` [T/world, K] token shard, ``w_local`` [N/world, K]; returns [T, N/world]."""
    return _ColumnParallel.apply(x_shard, w_local, tp, main_grad)


def row_parallel_linear(x: torch.Tensor, w_local: torch.Tensor, tp: TensorParallel,
                        main_grad: torch.Tensor | None = None) -> torch.Tensor:
    """``x`` [T, K/world], ``w_local`` [N, K/world]; returns the token shard [T/world, N] of the summed product."""
    return _RowParallel.apply(x, w_local, tp, main_grad)
