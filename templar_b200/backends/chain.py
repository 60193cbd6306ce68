"""Chain back-ends: the block clock, the metagraph and bucket commitments.

The reference talks to a Bittensor subtensor (src/tplr/chain.py:39-85).  That network is one
option here (``make_subtensor`` returns a ``bittensor.subtensor`` when the config names a network; a missing
``bittensor`` package is then an error, never a silent fallback); :class:`StaticChain` is the offline replacement: a metagraph described by a dict /
JSON file, commitments kept in memory (or in a shared JSON file for multi-process runs), and a
block counter derived from wall time (``block_time`` seconds per block) or advanced by hand.
"""

from __future__ import annotations

import json
import os
import threading
import time
from pathlib import Path
from types import SimpleNamespace

import torch

from ..logging import logger


class StaticMetagraph:
    def __init__(self, n: int = 8, stakes=None, hotkeys=None, validator_uids=(0,)):
        self.uids = torch.arange(n)
        self.hotkeys = list(hotkeys) if hotkeys else [f"hotkey-{i}" for i in range(n)]
        if stakes is None:
            stakes = [100000.0 if i in validator_uids else 10.0 for i in range(n)]
        self.S = torch.tensor(stakes, dtype=torch.float32)
        self.n = n
        self.block = 0

    def sync(self, subtensor=None, lite: bool = True):
        if subtensor is not None:
            self.block = subtensor.block
        return self


class StaticChain:
    """Subtensor stand-in. ``block`` grows with wall time unless ``manual`` is set."""

    def __init__(self, netuid: int = 3, n: int = 8, block_time: float = 12.0, genesis: float | None = None,
                 state_file: str | None = None, manual: bool = False, **metagraph_kw):
        self.netuid, self.block_time, self.manual = netuid, block_time, manual
        self.genesis = time.time() if genesis is None else genesis
        self._manual_block = 0
        self._metagraph = StaticMetagraph(n, **metagraph_kw)
        self._commit: dict[int, str] = {}
        self._weights: dict[int, tuple] = {}
        self.state_file = Path(state_file) if state_file else None
        self._lock = threading.Lock()
        self.substrate = SimpleNamespace(close=lambda: None, initialize=lambda: None)

    # -- clock --------------------------------------------------------------------------
    @property
    def block(self) -> int:
        if self.manual:
            return self._manual_block
        return int((time.time() - self.genesis) / self.block_time)

    def advance(self, n: int = 1) -> int:
        self._manual_block += n
        return self._manual_block

    def get_current_block(self) -> int:
        return self.block

    def block_timestamp(self, block: int) -> float:
        return self.genesis + block * self.block_time

    def metagraph(self, netuid: int | None = None):
        return self._metagraph

    # -- commitments ----------------------------------------------------------------------
    def _load(self):
        if self.state_file and self.state_file.exists():
            try:
                d = json.loads(self.state_file.read_text())
                self._commit.update({int(k): v for k, v in d.get("commitments", {}).items()})
            except Exception as e:  # noqa: BLE001
                logger.warning(f"static chain: state file {self.state_file} is unreadable ({e}); starting empty")

    def commit(self, wallet, netuid: int, data: str) -> None:
        uid = self._metagraph.hotkeys.index(wallet.hotkey.ss58_address)
        with self._lock:
            self._load()
            self._commit[uid] = data
            if self.state_file:
                self.state_file.parent.mkdir(parents=True, exist_ok=True)
                tmp = self.state_file.with_suffix(f".tmp{os.getpid()}")
                tmp.write_text(json.dumps({"commitments": self._commit}))
                os.replace(tmp, self.state_file)

    def get_commitment(self, netuid: int, uid: int) -> str:
        self._load()
        return self._commit.get(int(uid), "")

    def all_commitments(self) -> dict[int, str]:
        self._load()
        return dict(self._commit)

    def set_weights(self, wallet=None, netuid=None, uids=None, weights=None, **_) -> tuple[bool, str]:
        self._weights[self.block] = (list(map(int, uids)), [float(w) for w in weights])
        return True, "ok"


class StaticWallet:
    def __init__(self, hotkey: str = "hotkey-0", name: str = "static"):
        self.name = name
        self.hotkey = SimpleNamespace(ss58_address=hotkey)
        self.hotkey_str = hotkey


def make_subtensor(config):
    """The static chain for ``static`` / ``offline`` (or no) network, else a ``bittensor.subtensor`` for that network."""
    network = getattr(getattr(config, "subtensor", None), "network", None) or getattr(config, "network", None)
    if network and network not in ("static", "offline", "local-static"):
        try:
            import bittensor as bt
        except ImportError as e:
            # never fall back silently: a node asked to join a real network must not run against a private chain
            raise RuntimeError(f"network '{network}' was requested but the bittensor package is not installed; "
                               f"use --network static for an offline run") from e
        try:
            return bt.subtensor(config=config)
        except Exception:  # noqa: BLE001  (a plain namespace instead of a bittensor config object)
            return bt.subtensor(network=network)
    kw = dict(getattr(config, "static_chain", {}) or {})
    return StaticChain(netuid=getattr(config, "netuid", 3), **kw)
