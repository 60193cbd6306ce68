"""Burn-only validator: every ``WEIGHT_INTERVAL`` blocks set 100 % of the weight on the burn uid.

Parity: the reference's neurons/burn.py:11-90.  ``python neurons/burn.py --netuid 268 [--network static]``.
"""

from __future__ import annotations

import argparse
import os
import sys
import time
from types import SimpleNamespace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from templar_b200.backends.chain import StaticWallet, make_subtensor  # noqa: E402

BURN_UID = 1
WEIGHT_INTERVAL = 360


def get_config(argv=None) -> SimpleNamespace:
    p = argparse.ArgumentParser(description="Burn-only validator script")
    p.add_argument("--netuid", type=int, default=268)
    p.add_argument("--network", type=str, default="static")
    p.add_argument("--wallet-hotkey", type=str, default="hotkey-0")
    p.add_argument("--poll-seconds", type=float, default=12.0)
    p.add_argument("--max-iterations", type=int, default=0, help="0 = run until interrupted")
    return SimpleNamespace(**vars(p.parse_args(argv)))


def run(config, subtensor=None, wallet=None, sleep=time.sleep) -> int:
    """Returns the number of successful weight sets (the loop ends after ``max_iterations`` polls)."""
    subtensor = subtensor or make_subtensor(config)
    wallet = wallet or StaticWallet(config.wallet_hotkey)
    metagraph = subtensor.metagraph(config.netuid)
    my_uid = metagraph.hotkeys.index(wallet.hotkey.ss58_address)
    tplr.logger.info(f"Running burn on UID {my_uid}, netuid {config.netuid}: 100% weight to UID {BURN_UID} "
                     f"every {WEIGHT_INTERVAL} blocks")
    last_set, sets, it = 0, 0, 0
    while not config.max_iterations or it < config.max_iterations:
        it += 1
        try:
            block = subtensor.block
            if block - last_set >= WEIGHT_INTERVAL:
                ok, msg = subtensor.set_weights(wallet=wallet, netuid=config.netuid, uids=[BURN_UID], weights=[1.0],
                                                wait_for_inclusion=True)
                if ok:
                    last_set, sets = block, sets + 1
                    tplr.logger.info(f"Weights set successfully at block {block}")
                else:
                    tplr.logger.warning(f"Failed to set weights: {msg}")
            elif it % 10 == 0:
                tplr.logger.info(f"Block {block} | next weight set in {max(0, WEIGHT_INTERVAL - (block - last_set))} blocks")
            sleep(config.poll_seconds)
        except KeyboardInterrupt:
            break
        except Exception as e:  # noqa: BLE001
            tplr.logger.error(f"Error: {e}")
            sleep(config.poll_seconds)
    return sets


def main():
    run(get_config())


if __name__ == "__main__":
    main()
