"""B200-native framework with the capabilities and flat public API of templar (``tplr``).

``import templar_b200 as tplr`` (or ``import tplr``) exposes ``tplr.Comms``,
``tplr.prepare_gradient_dict``, ``tplr.DCPCheckpointer``, ``tplr.MinerSampler`` … like the
reference's package root (src/tplr/__init__.py:22-40).
"""

__version__ = "2.1.28"

from . import compress, config, decos, distributed, exceptions, logging, schemas  # noqa: E402,F401
from .chain import *  # noqa: E402,F401,F403
from .chain import ChainManager  # noqa: E402,F401
from .comms import Comms  # noqa: E402,F401
from .compress import *  # noqa: E402,F401,F403
from .dcp_checkpoint import DCPCheckpointer  # noqa: E402,F401
from .hparams import load_hparams  # noqa: E402,F401
from .logging import P, T, debug, log_with_context, logger, setup_loki_logger, trace_on  # noqa: E402,F401
from .neurons import *  # noqa: E402,F401,F403
from .schemas import Bucket, CommsGetResult  # noqa: E402,F401
from .dataset import DatasetLoader, SubsetLoader  # noqa: E402,F401
from .sharded_dataset import SharedShardedDataset, ShardedDatasetManager, SyntheticDataset, compute_shard_state  # noqa: E402,F401
from .sharded_sampler import EvalSampler, MinerSampler  # noqa: E402,F401
from .wandb_ops import initialize_wandb  # noqa: E402,F401
from .metrics import MetricsLogger  # noqa: E402,F401
from . import backends, metrics, model_factory, muon, profilers, wandb_ops  # noqa: E402,F401
