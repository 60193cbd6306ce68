"""Process-group helper (``dist_helper`` singleton): bootstrap, consensus flags, object
collectives and the parameter snapshot / pseudo-gradient restore.

API parity with the reference's ``DistributedHelper`` (src/tplr/distributed.py:35-549).  Two
differences in how the work is done:

* flags and scalar reductions share one implementation (``_reduce_flag``) that never raises;
* ``get_offloaded_params`` / ``restore_offloaded_params`` keep the snapshot wherever it is cheapest:
  for models attached to a :class:`~templar_b200.parallel.window_engine.WindowEngine` the snapshot
  is the engine's HBM-resident ``theta0`` and the restore is fused into the compress and outer
  step kernels; for any other model the generic path copies to reusable (pinned when CUDA is
  present) host buffers on a side stream and rebuilds ``p.grad = saved - p; p <- saved``.
"""

from __future__ import annotations

import os
import time
from contextlib import nullcontext
from datetime import timedelta
from typing import Any

import torch
import torch.distributed as dist

from .logging import logger


class DistributedHelper:
    def __init__(self):
        self.rank = int(os.getenv("RANK", 0))
        self.world_size = int(os.getenv("WORLD_SIZE", 1))
        self.local_rank = int(os.getenv("LOCAL_RANK", 0))
        self.is_master = self.rank == 0
        self.device = None

    # -- bootstrap -----------------------------------------------------------------------
    def init_process_group(self, backend: str = "nccl", timeout_minutes: int = 45) -> None:
        self.__init__()
        if dist.is_initialized() or self.world_size <= 1:
            if self.device is None:
                self.device = (torch.device(f"cuda:{self.local_rank}") if torch.cuda.is_available()
                               else torch.device("cpu"))
            return
        if backend == "nccl" and not torch.cuda.is_available():
            backend = "gloo"
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device(f"cuda:{self.local_rank}")
            kwargs["device_id"] = self.device
        else:
            self.device = torch.device("cpu")
        dist.init_process_group(backend=backend, init_method="env://", timeout=timedelta(minutes=timeout_minutes),
                                rank=self.rank, world_size=self.world_size, **kwargs)
        logger.info(f"[Distributed] rank={self.rank}/{self.world_size} local_rank={self.local_rank} "
                    f"backend={backend} device={self.device}")

    def solo(self) -> tuple[int, int]:
        """Co-located nodes: the ranks of the process group are independent nodes (one uid each) that only share peer
        memory.  From here on this helper answers as a single-rank node (no collective of a node's own protocol runs
        across the group); returns ``(group_rank, group_world_size)`` for the code that does use the group."""
        self.group_rank, self.group_world_size = self.rank, self.world_size
        self.rank, self.world_size, self.is_master = 0, 1, True
        return self.group_rank, self.group_world_size

    def destroy_process_group(self) -> None:
        if (self.world_size > 1 or getattr(self, "group_world_size", 1) > 1) and dist.is_initialized():
            dist.destroy_process_group()

    def is_distributed(self) -> bool:
        return dist.is_available() and dist.is_initialized() and self.world_size > 1

    # -- scalar / flag collectives ---------------------------------------------------------
    def _reduce_flag(self, value: bool, op, device, tag: str, on_error: bool) -> bool:
        if not self.is_distributed():
            return bool(value)
        try:
            t = torch.tensor([1 if value else 0], device=device, dtype=torch.int32)
            dist.all_reduce(t, op=op)
            return bool(int(t.item()))
        except Exception as e:  # noqa: BLE001
            logger.error(f"[Distributed] flag reduce '{tag}' failed: {e}")
            return on_error

    def should_continue(self, local_has_batch: bool, device) -> bool:
        if not self.is_distributed():
            return local_has_batch
        return self._reduce_flag(local_has_batch, dist.ReduceOp.MIN, device, "should_continue", False)

    def all_ok(self, ok: bool, device, tag: str = "") -> bool:
        return self._reduce_flag(ok, dist.ReduceOp.MIN, device, tag, False)

    def any_ok(self, ok: bool, device, tag: str = "") -> bool:
        return self._reduce_flag(ok, dist.ReduceOp.MAX, device, tag, False)

    def all_agree(self, agree: bool, device, tag: str = "") -> bool:
        return self._reduce_flag(agree, dist.ReduceOp.MIN, device, tag, bool(agree))

    def all_reduce_flag(self, ok: bool, device, tag: str = "") -> bool:
        return self._reduce_flag(ok, dist.ReduceOp.MIN, device, tag, False)

    def ddp_reduce(self, value, op=dist.ReduceOp.SUM, device=None) -> float:
        if not self.is_distributed():
            return float(value.item() if isinstance(value, torch.Tensor) else value)
        device = device or self.device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        t = (value.detach().to(device=device, dtype=torch.float32).clone() if isinstance(value, torch.Tensor)
             else torch.tensor(float(value), device=device))
        if op == dist.ReduceOp.AVG and dist.get_backend() == "gloo":
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            t /= self.world_size
        else:
            dist.all_reduce(t, op=op)
        return float(t.item())

    # -- barriers ---------------------------------------------------------------------------
    def barrier(self, device_ids: list | None = None) -> None:
        if not self.is_distributed():
            return
        if device_ids is not None and dist.get_backend() == "nccl":
            dist.barrier(device_ids=device_ids)
        else:
            dist.barrier()

    def safe_barrier(self, tag: str = "", local_rank: int | None = None) -> bool:
        """Barrier that reports failure instead of raising."""
        if not self.is_distributed():
            return True
        try:
            if dist.get_backend() == "nccl" and torch.cuda.is_available():
                dist.barrier(device_ids=[self.local_rank if local_rank is None else local_rank])
            else:
                dist.barrier()
            return True
        except Exception as e:  # noqa: BLE001
            logger.error(f"[Distributed] barrier '{tag}' failed: {e}")
            return False

    # -- tensors / objects --------------------------------------------------------------------
    def broadcast(self, tensor: torch.Tensor, src: int = 0) -> None:
        if self.is_distributed():
            dist.broadcast(tensor, src=src)

    def gather_object(self, obj: Any, object_list: list | None = None, dst: int = 0) -> list | None:
        if not self.is_distributed():
            return [obj] if self.rank == dst else None
        if self.rank == dst and object_list is None:
            object_list = [None] * self.world_size
        dist.gather_object(obj, object_list if self.rank == dst else None, dst=dst)
        return object_list if self.rank == dst else None

    def all_gather_object(self, obj: Any, object_list: list | None = None) -> list:
        if not self.is_distributed():
            return [obj]
        if object_list is None:
            object_list = [None] * self.world_size
        dist.all_gather_object(object_list, obj)
        return object_list

    # -- parameter snapshot / pseudo-gradient ---------------------------------------------------
    @staticmethod
    def _model_device(model: torch.nn.Module) -> torch.device:
        return next(model.parameters()).device

    def _get_offload_stream(self, model):
        if not torch.cuda.is_available() or self._model_device(model).type != "cuda":
            return None
        s = getattr(model, "_offload_stream", None)
        if s is None:
            s = torch.cuda.Stream(device=self._model_device(model))
            model._offload_stream = s
        return s

    @staticmethod
    def _local(p):
        to_local = getattr(p, "to_local", None)
        return to_local() if callable(to_local) else p

    def get_offloaded_params(self, model: torch.nn.Module) -> tuple:
        """Snapshot the local parameters into reusable host buffers (async D2H on a side stream)."""
        engine = getattr(model, "_window_engine", None)
        if engine is not None:
            engine.snapshot()
            return ["engine"], [{"engine": True}]
        stream = self._get_offload_stream(model)
        t0 = time.time()
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        saved, specs = [], []
        with torch.no_grad(), (torch.cuda.stream(stream) if stream is not None else nullcontext()):
            for p in model.parameters():
                src = self._local(p).detach()
                buf = getattr(p, "_cpu_offload_buf", None)
                if buf is None or buf.shape != src.shape or buf.dtype != src.dtype:
                    buf = torch.empty(src.shape, dtype=src.dtype, device="cpu", pin_memory=src.is_cuda)
                    p._cpu_offload_buf = buf
                buf.copy_(src, non_blocking=True)
                saved.append(buf)
                specs.append({"is_dtensor": src is not p and hasattr(p, "device_mesh"),
                              "device_mesh": getattr(p, "device_mesh", None), "placements": getattr(p, "placements", None),
                              "local_shape": tuple(src.shape), "dtype": str(src.dtype).replace("torch.", "")})
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
            stream.synchronize()
        logger.info(f"[ParamOffload] snap {len(saved)} params in {time.time() - t0:.3f}s")
        return saved, specs

    def restore_offloaded_params(self, model: torch.nn.Module, params_offloaded: list, param_specs: list) -> None:
        """``p.grad <- saved - p`` (the window's pseudo-gradient) and ``p <- saved``."""
        if params_offloaded and isinstance(params_offloaded[0], str):
            return  # engine snapshot: delta and restore are fused into the compress / outer-step kernels
        stream = self._get_offload_stream(model)
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        t0 = time.time()
        with torch.no_grad(), (torch.cuda.stream(stream) if stream is not None else nullcontext()):
            for (saved, meta), p in zip(zip(params_offloaded, param_specs), model.parameters()):
                local = self._local(p)
                if meta.get("is_dtensor") and hasattr(p, "device_mesh"):
                    from torch.distributed.tensor import DTensor

                    g = torch.empty_like(local)
                    g.copy_(saved, non_blocking=True)
                    g.sub_(local)
                    local.add_(g)
                    p.grad = DTensor.from_local(g, device_mesh=meta["device_mesh"], placements=meta["placements"],
                                                run_check=False)
                    continue
                if p.grad is None or p.grad.shape != local.shape or p.grad.device != local.device:
                    p.grad = torch.empty_like(local)
                p.grad.copy_(saved, non_blocking=True)
                p.grad.sub_(local)
                local.add_(p.grad)
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
            stream.synchronize()
        logger.info(f"[ParamRestore] restored {len(params_offloaded)} params in {time.time() - t0:.3f}s")


dist_helper = DistributedHelper()
