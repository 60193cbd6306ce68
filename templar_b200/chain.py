"""Chain manager: block/window tracking, bucket commitments, peer bookkeeping.

Parity with the reference's ``ChainManager`` (src/tplr/chain.py:36-410): a commitment is the
128-character string ``account_id[32] ‖ access_key_id[32] ‖ secret_access_key[64]`` (the account id
doubles as the bucket name), commitments are re-fetched every ``fetch_interval`` seconds in a
background task, ``update_peers_with_buckets`` keeps ``eval_peers`` (active peers whose stake is at
most 20000) and ``inactive_peers`` (previously evaluated, no longer active).  The chain itself is a
pluggable back-end (:mod:`templar_b200.backends.chain`): Bittensor when available, a static
offline chain otherwise.
"""

from __future__ import annotations

import asyncio
from collections import defaultdict
from types import SimpleNamespace

import numpy as np
import torch

from .backends.chain import make_subtensor
from .logging import logger
from .schemas import Bucket

COMMITMENT_LEN = 128


def encode_commitment(bucket: Bucket) -> str:
    s = bucket.account_id + bucket.access_key_id + bucket.secret_access_key
    if len(s) != COMMITMENT_LEN:
        raise ValueError(f"Commitment is {len(s)} characters but must be {COMMITMENT_LEN} "
                         f"(account id 32, access key id 32, secret 64)")
    return s


def decode_commitment(s: str) -> Bucket:
    if len(s) != COMMITMENT_LEN:
        raise ValueError(f"Commitment '{s[:8]}…' is of length {len(s)} but should be of length {COMMITMENT_LEN}.")
    try:
        return Bucket(name=s[:32], account_id=s[:32], access_key_id=s[32:64], secret_access_key=s[64:])
    except Exception as e:  # pydantic ValidationError
        raise ValueError(f"Invalid data in commitment: {e}") from e


class ChainManager:
    def __init__(self, config, hparams=None, fetch_interval: int = 600, wallet=None, bucket: Bucket | None = None,
                 subtensor=None):
        self.config = config
        self.netuid = getattr(config, "netuid", 3)
        self.hparams = hparams or SimpleNamespace()
        self.subtensor = subtensor if subtensor is not None else make_subtensor(config)
        self.metagraph = self.subtensor.metagraph(self.netuid)
        self.current_block = 0
        self.current_window = 0
        self.window_duration = getattr(self.hparams, "blocks_per_window", 1)
        self.window_time = 0
        self.window_seeds: dict = {}
        self.block_event = asyncio.Event()
        self.new_window_event = asyncio.Event()
        self.commitments: dict[int, Bucket] = {}
        self.peers: list[int] = []
        self.eval_peers: dict[int, int] = defaultdict(int)
        self.active_peers: set[int] = set()
        self.inactive_peers: set[int] = set()
        self.fetch_interval = fetch_interval
        self._fetch_task = None
        self.wallet, self.bucket = wallet, bucket

    # -- background refresh -------------------------------------------------------------------
    def start_commitment_fetcher(self) -> None:
        if self._fetch_task is None:
            self._fetch_task = asyncio.create_task(self._fetch_commitments_periodically())

    async def _fetch_commitments_periodically(self) -> None:
        while True:
            try:
                await asyncio.to_thread(lambda: self.metagraph.sync(subtensor=self.subtensor))
                got = await self.get_commitments()
                if got:
                    self.commitments = got
            except Exception as e:  # noqa: BLE001
                logger.error(f"Error fetching commitments: {e}")
                self._reconnect()
            await asyncio.sleep(self.fetch_interval)

    def _reconnect(self) -> None:
        sub = getattr(self.subtensor, "substrate", None)
        if sub is not None:
            try:
                sub.close()
                sub.initialize()
            except Exception as e:  # noqa: BLE001
                logger.debug(f"substrate reconnect failed: {e}")

    # -- commitments ----------------------------------------------------------------------------
    def get_bucket(self, uid: int) -> Bucket | None:
        return self.commitments.get(uid)

    def get_all_buckets(self) -> dict[int, Bucket | None]:
        return {int(uid): self.get_bucket(int(uid)) for uid in self._uids()}

    def commit(self, wallet, bucket: Bucket) -> None:
        self.subtensor.commit(wallet, self.netuid, encode_commitment(bucket))
        logger.info(f"Committed bucket configuration to chain for hotkey {wallet.hotkey.ss58_address}")

    def try_commit(self, wallet, bucket: Bucket) -> None:
        """Commit ``bucket`` unless the chain already holds the same commitment for this wallet."""
        try:
            uid = self.metagraph.hotkeys.index(wallet.hotkey.ss58_address)
            existing = self.get_commitment(uid)
            if existing == bucket:
                logger.info("Bucket commitment already on chain and up to date")
                return
        except Exception as e:  # noqa: BLE001
            logger.info(f"No usable commitment on chain yet ({e})")
        self.commit(wallet, bucket)

    def get_commitment(self, uid: int) -> Bucket:
        try:
            s = self.subtensor.get_commitment(self.netuid, uid)
        except Exception as e:  # noqa: BLE001
            raise Exception(f"Couldn't get commitment from uid {uid} because {e}") from e
        return decode_commitment(s)

    async def get_commitments(self, block: int | None = None) -> dict[int, Bucket]:
        try:
            if hasattr(self.subtensor, "all_commitments"):
                raw = {uid: s for uid, s in self.subtensor.all_commitments().items()}
            else:
                raw = self._query_commitment_map(block)
        except Exception as e:  # noqa: BLE001
            logger.error(f"commitment query failed: {e}")
            self._reconnect()
            return {}
        out = {}
        for uid, s in raw.items():
            try:
                out[int(uid)] = decode_commitment(s)
            except ValueError as e:
                logger.error(f"Invalid commitment for UID {uid}: {e}")
        return out

    @staticmethod
    def decode_metadata(encoded_ss58: tuple, metadata: dict, decode_account_id=None) -> tuple[str, str]:
        """(hotkey address, commitment text) of one entry of the chain's commitment map: the key's first element is the
        account id, the text sits as a byte tuple under the only key of ``info.fields[0][0]``
        (reference: src/tplr/chain.py:256-262)."""
        if decode_account_id is None:
            from bittensor.core.chain_data import decode_account_id  # optional dependency
        commitment = metadata["info"]["fields"][0][0]
        return decode_account_id(encoded_ss58[0]), bytes(commitment[next(iter(commitment.keys()))][0]).decode()

    def _query_commitment_map(self, block):
        """Bittensor path: walk the Commitments.CommitmentOf map and key it by uid."""
        from bittensor.core.chain_data import decode_account_id  # optional dependency

        substrate = self.subtensor.substrate
        result = substrate.query_map(module="Commitments", storage_function="CommitmentOf", params=[self.netuid],
                                     block_hash=None if block is None else substrate.get_block_hash(block))
        hotkey_to_uid = dict(zip(self.metagraph.hotkeys, self._uids()))
        raw = {}
        for key, value in result:
            try:
                ss58, data = self.decode_metadata(key, value.value, decode_account_id)
            except Exception as e:  # noqa: BLE001
                logger.error(f"Failed to decode commitment metadata: {e}")
                continue
            if ss58 in hotkey_to_uid:
                raw[int(hotkey_to_uid[ss58])] = data
        return raw

    async def fetch_commitments(self) -> None:
        got = await self.get_commitments()
        if got:
            self.commitments = got
        else:
            logger.warning("No commitments fetched.")

    async def get_bucket_for_neuron(self, wallet) -> Bucket | None:
        try:
            return self.get_bucket(self.metagraph.hotkeys.index(wallet.hotkey.ss58_address))
        except ValueError:
            logger.warning(f"Hotkey {wallet.hotkey.ss58_address} not found in metagraph")
            return None

    # -- metagraph helpers ------------------------------------------------------------------------
    def _uids(self) -> list[int]:
        u = self.metagraph.uids
        return [int(x) for x in (u.tolist() if isinstance(u, (np.ndarray, torch.Tensor)) else u)]

    def get_hotkey(self, uid: int) -> str | None:
        uids = self._uids()
        hk = self.metagraph.hotkeys
        hk = hk.tolist() if isinstance(hk, (np.ndarray, torch.Tensor)) else hk
        return hk[uids.index(uid)] if uid in uids else None

    def update_peers_with_buckets(self) -> None:
        stakes = self.metagraph.S.tolist() if hasattr(self.metagraph.S, "tolist") else list(self.metagraph.S)
        uid_to_stake = dict(zip(self._uids(), stakes))
        active = {int(u) for u in self.active_peers}
        self.inactive_peers = set(self.eval_peers.keys()) - active
        logger.info(f"Newly inactive peers: {self.inactive_peers}")
        if not active:
            logger.warning("No active peers found. Skipping update.")
            return
        self.eval_peers = {uid: self.eval_peers.get(uid, 1) for uid in active
                           if uid in uid_to_stake and uid_to_stake[uid] <= 20000}
        logger.info(f"Total evaluation peers: {len(self.eval_peers)}; inactive: {len(self.inactive_peers)}")
