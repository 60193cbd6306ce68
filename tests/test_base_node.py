"""BaseNode: block listener with a flaky subscription, window bookkeeping, timestamp retries, shutdown."""

import asyncio
import signal
import threading
from types import SimpleNamespace

import pytest

import neurons.base_node as bn
from neurons.base_node import BaseNode


class _Node(BaseNode):
    def __init__(self, blocks_per_window=10):
        super().__init__()
        self.hparams = SimpleNamespace(blocks_per_window=blocks_per_window)
        self.config = SimpleNamespace()

    async def run(self):
        return None


class _FlakySubstrate:
    """subscribe_block_headers raises for the first ``drops`` calls, then feeds ``blocks`` and raises again."""

    def __init__(self, node, drops, blocks):
        self.node, self.drops, self.blocks, self.calls, self.closed, self.inits = node, drops, blocks, 0, 0, 0

    def initialize(self):
        self.inits += 1

    def close(self):
        self.closed += 1

    def subscribe_block_headers(self, handler):
        self.calls += 1
        if self.calls <= self.drops:
            raise ConnectionError("websocket closed")
        for b in self.blocks:
            handler({"header": {"number": b}})
        self.node.stop_event.set()                       # host-side end of the test
        raise ConnectionError("stream ended")


def test_block_listener_reconnects_with_exponential_backoff(monkeypatch):
    node = _Node()
    sleeps = []
    monkeypatch.setattr(bn.time, "sleep", lambda s: sleeps.append(s))
    sub = SimpleNamespace()
    sub.substrate = _FlakySubstrate(node, drops=3, blocks=[7, 12, 25])
    node.subtensor_rpc = sub
    t = threading.Thread(target=node.block_listener, daemon=True)
    t.start()
    t.join(10)
    assert not t.is_alive()
    assert sleeps[:3] == [1, 2, 4]                        # back-off doubles while the subscription keeps dropping
    assert sub.substrate.calls == 4 and sub.substrate.closed >= 4 and sub.substrate.inits == 4
    assert node.current_block == 25 and node.current_window == 2


def test_on_block_updates_window_and_notifies_waiters():
    async def go():
        node = _Node(blocks_per_window=5)
        node.window_changed = asyncio.Event()
        node._notify_loop = asyncio.get_running_loop()
        node.comms = SimpleNamespace(current_window=0)
        waiter = asyncio.create_task(node.wait_until_window(2))
        await asyncio.sleep(0.01)
        threading.Thread(target=lambda: [node._on_block(b) for b in (3, 6, 11)], daemon=True).start()
        await asyncio.wait_for(waiter, 5)
        return node

    node = asyncio.run(go())
    assert node.current_window == 2 and node.comms.current_window == 2 and node.current_block == 11


def test_query_block_timestamp_retries_then_gives_up(monkeypatch):
    node = _Node()
    monkeypatch.setattr(bn.time, "sleep", lambda s: None)
    calls = {"n": 0}

    class _Sub:
        substrate = SimpleNamespace(close=lambda: None, initialize=lambda: None)

        def query_module(self, module, name, block=None):
            calls["n"] += 1
            if calls["n"] < 3:
                raise RuntimeError("rpc down")
            return SimpleNamespace(value=1_700_000_000_000 + block)

    node.subtensor_client = _Sub()
    assert node.query_block_timestamp(5) == pytest.approx(1_700_000_000.005)
    assert calls["n"] == 3

    class _Dead(_Sub):
        def query_module(self, *a, **k):
            raise RuntimeError("rpc down")

    node.subtensor_client = _Dead()
    assert node.query_block_timestamp(5, retries=2) is None
    node.subtensor_client = SimpleNamespace(block_timestamp=lambda b: 12.0 * b)     # static chain: direct answer
    assert node.query_block_timestamp(4) == 48.0


def test_graceful_shutdown_flushes_uploads_and_cancels_tasks():
    async def go():
        node = _Node()
        flushed = []

        async def flush():
            flushed.append(True)

        node.ckpt = SimpleNamespace(flush_background_uploads=flush)
        task = asyncio.create_task(asyncio.sleep(60))
        node._bg_tasks.add(task)
        closed = []
        node.subtensor_rpc = SimpleNamespace(close=lambda: closed.append("rpc"))
        node.subtensor_client = SimpleNamespace(close=lambda: closed.append("client"))
        await node._graceful_shutdown(signal.SIGTERM)
        return node, flushed, task, closed

    node, flushed, task, closed = asyncio.run(go())
    assert node.stop_event.is_set() and flushed == [True] and task.cancelled() and closed == ["rpc", "client"]


def test_profiler_config_only_when_requested(tmp_path):
    node = _Node()
    assert node._profiler_config() is None
    node.config = SimpleNamespace(profile_iters=2, profile_dir=str(tmp_path))
    node.rank = 1
    cfg = node._profiler_config()
    assert cfg["record_shapes"] and (tmp_path / "rank_1").is_dir()
