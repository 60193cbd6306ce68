"""Node runtime shared by every neuron: asyncio main, signals, graceful shutdown, the block
clock thread and window waiting.

Parity: the reference's neurons/base_node.py:24-296.  The block source is pluggable: with a
Bittensor subtensor the listener subscribes to block headers and reconnects with exponential
back-off (1 s doubling to 60 s); with the offline :class:`~templar_b200.backends.chain.StaticChain`
it polls the wall-clock-derived block number.  Either way ``current_block`` / ``current_window`` are
updated from a daemon thread and ``window_changed`` is set on the event loop.
"""

from __future__ import annotations

import abc
import asyncio
import functools
import os
import signal
import threading
import time
from types import SimpleNamespace
from typing import Any

import templar_b200 as tplr
from templar_b200.backends.chain import StaticChain, make_subtensor
from templar_b200.distributed import dist_helper


class BaseNode(abc.ABC):
    world_size: int = 1
    config: Any = None
    hparams: SimpleNamespace

    def __init__(self):
        self.stop_event = asyncio.Event()
        self._bg_tasks: set[asyncio.Task] = set()
        self._threads: list[threading.Thread] = []
        self.window_changed: asyncio.Event | None = None
        self._notify_loop: asyncio.AbstractEventLoop | None = None
        self.current_block = 0
        self.current_window = 0
        self.subtensor_rpc = None
        self.subtensor_client = None
        self._prof = None
        self._prof_config = None

    # -- main -----------------------------------------------------------------------------
    async def main(self):
        loop = asyncio.get_running_loop()
        self._setup_signal_handlers(loop)
        self.window_changed = asyncio.Event()
        self._notify_loop = loop
        t = threading.Thread(target=self.block_listener, name="blocks", daemon=True)
        t.start()
        self._threads.append(t)
        self._prof_config = self._profiler_config()
        try:
            await self.run()
        except Exception:  # noqa: BLE001
            tplr.logger.error("Unhandled exception in run()", exc_info=True)
        finally:
            if not self.stop_event.is_set():
                await self._graceful_shutdown(signal.SIGTERM)

    def _profiler_config(self):
        iters = int(getattr(self.config, "profile_iters", 0) or 0)
        if iters <= 0:
            return None
        import torch.profiler as tp

        out = f"{getattr(self.config, 'profile_dir', './log/profiler')}/rank_{getattr(self, 'rank', 0)}"
        os.makedirs(out, exist_ok=True)
        return {"activities": [tp.ProfilerActivity.CPU, tp.ProfilerActivity.CUDA],
                "schedule": tp.schedule(wait=0, warmup=1, active=iters, repeat=1),
                "on_trace_ready": tp.tensorboard_trace_handler(out), "record_shapes": True, "profile_memory": True,
                "with_stack": True}

    @abc.abstractmethod
    async def run(self):
        raise NotImplementedError

    def gather_wait_seconds(self) -> float:
        """How long a gather waits for peers' uploads.  On a network the upload-time window ends the wait; an offline
        run has no such window, and a peer that skipped a window would otherwise hold everyone for the whole
        time-out: there the wait is one window long (blocks per window x block time), at least two seconds."""
        limit = float(getattr(self, "gather_timeout", 90))
        if getattr(self.config, "local", False):
            window_s = float(getattr(self.hparams, "blocks_per_window", 7)) * float(getattr(self.config, "block_time", 12.0))
            limit = min(limit, max(2.0, window_s))
        return limit

    # -- windows ----------------------------------------------------------------------------
    async def wait_until_window(self, target_window: int) -> None:
        evt = self.window_changed
        if evt is not None and evt.is_set():
            evt.clear()
        while not self.stop_event.is_set():
            if self.current_window >= target_window:
                return
            bpw = self.hparams.blocks_per_window
            remaining = (target_window - self.current_window) * bpw - self.current_block % bpw
            eta = max(0, remaining * 12)
            tplr.logger.info(f"waiting for window {target_window} (~{eta // 60} m {eta % 60:02d} s, {remaining} blocks)")
            if evt is None:
                await asyncio.sleep(0.5)
            else:
                try:
                    await asyncio.wait_for(evt.wait(), timeout=5.0)
                except asyncio.TimeoutError:
                    pass
                evt.clear()

    def _on_block(self, number: int) -> None:
        self.current_block = int(number)
        new_window = self.current_block // self.hparams.blocks_per_window
        if new_window != self.current_window:
            self.current_window = new_window
            if hasattr(self, "comms"):
                self.comms.current_window = new_window
            tplr.logger.info(f"window -> {new_window}")
            if self.window_changed is not None and self._notify_loop is not None:
                self._notify_loop.call_soon_threadsafe(self.window_changed.set)

    def block_listener(self):
        """Daemon thread: feeds ``_on_block`` until ``stop_event`` is set."""
        backoff, max_backoff = 1, 60
        if self.subtensor_rpc is None:
            self.subtensor_rpc = getattr(self, "subtensor", None) or make_subtensor(self.config)
        sub = self.subtensor_rpc
        if isinstance(sub, StaticChain) or not hasattr(getattr(sub, "substrate", None), "subscribe_block_headers"):
            while not self.stop_event.is_set():
                try:
                    self._on_block(sub.block)
                except Exception as e:  # noqa: BLE001
                    tplr.logger.error(f"block-poll err: {e}")
                time.sleep(min(0.25, getattr(sub, "block_time", 1.0) / 4))
            return

        def handler(event):
            try:
                self._on_block(int(event["header"]["number"]))
            except Exception as e:  # noqa: BLE001
                tplr.logger.error(f"block-handler err: {e}")

        while not self.stop_event.is_set():
            try:
                sub.substrate.initialize()
                sub.substrate.subscribe_block_headers(handler)
                backoff = 1
            except Exception as e:  # noqa: BLE001  (websocket closed, RPC errors …)
                if self.stop_event.is_set():
                    break
                tplr.logger.warning(f"block subscription dropped: {e} – retrying in {backoff}s")
            finally:
                try:
                    sub.substrate.close()
                except Exception:  # noqa: BLE001
                    pass
            time.sleep(backoff)
            backoff = min(backoff * 2, max_backoff)

    def query_block_timestamp(self, block: int, *, retries: int = 5, init_delay: float = 1.0,
                              max_delay: float = 60.0) -> float | None:
        """Unix time (s) of ``block`` or None; a separate client from the listener, exponential back-off."""
        if self.subtensor_client is None:
            self.subtensor_client = getattr(self, "subtensor", None) or make_subtensor(self.config)
        sub = self.subtensor_client
        if hasattr(sub, "block_timestamp"):
            return float(sub.block_timestamp(block))
        delay = init_delay
        for attempt in range(1, retries + 1):
            try:
                resp = sub.query_module("Timestamp", "Now", block=block)
                if resp is None or not hasattr(resp, "value"):
                    raise ValueError(f"Could not query timestamp for {block}")
                return int(resp.value) / 1000
            except Exception as e:  # noqa: BLE001
                tplr.logger.warning(f"[timestamp] block {block} attempt {attempt}/{retries} failed: {e}")
                if attempt == retries:
                    return None
                try:
                    sub.substrate.close()
                    sub.substrate.initialize()
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(delay)
                delay = min(delay * 2, max_delay)
        return None

    # -- shutdown ------------------------------------------------------------------------------
    def _setup_signal_handlers(self, loop: asyncio.AbstractEventLoop):
        for sig in (signal.SIGINT, signal.SIGTERM):
            try:
                loop.add_signal_handler(sig, functools.partial(self._spawn_shutdown, sig))
            except (NotImplementedError, RuntimeError):
                pass

    def _spawn_shutdown(self, sig):
        asyncio.create_task(self._graceful_shutdown(sig))

    async def _graceful_shutdown(self, sig):
        tplr.logger.warning(f"received {getattr(sig, 'name', sig)} – shutting down …")
        self.stop_event.set()
        ckpt = getattr(self, "ckpt", None)
        if ckpt is not None:
            await ckpt.flush_background_uploads()
        for task in list(self._bg_tasks):
            task.cancel()
        await asyncio.gather(*self._bg_tasks, return_exceptions=True)
        for th in self._threads:
            th.join(timeout=2)
        for sub in (self.subtensor_rpc, self.subtensor_client):
            close = getattr(sub, "close", None)
            if callable(close):
                try:
                    close()
                except Exception:  # noqa: BLE001
                    pass
        ex = getattr(self, "executor", None)
        if ex is not None:
            ex.shutdown(wait=False, cancel_futures=True)
        if hasattr(self, "world_size"):
            dist_helper.destroy_process_group()
        await asyncio.sleep(0.05)
        tplr.logger.info("shutdown complete")
