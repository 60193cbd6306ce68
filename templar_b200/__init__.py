"""B200-native framework with the capabilities and flat public API of templar (``tplr``).

``import templar_b200 as tplr`` (or ``import tplr``) exposes ``tplr.Comms``,
``tplr.prepare_gradient_dict``, ``tplr.DCPCheckpointer``, ``tplr.MinerSampler`` … like the
reference's package root (src/tplr/__init__.py:22-40).
"""

__version__ = "2.1.28"

from . import compress, config, decos, distributed, exceptions, logging, schemas  # noqa: E402,F401
from .chain import *  # noqa: E402,F401,F403
from .chain import ChainManager  # noqa: E402,F401
from .comms import (CF_REGION_NAME, CPU_COUNT, CPU_MAX_CONNECTIONS, LOCAL_TMP_DIR, PEERS_FILE_PREFIX, SAFE_BUCKET_RE,  # noqa: E402,F401
                    SAFE_KEY_RE, Comms)
from .compress import *  # noqa: E402,F401,F403
from .dcp_checkpoint import DCPCheckpointer  # noqa: E402,F401
from .hparams import DEFAULT_HPARAMS, create_namespace, load_hparams  # noqa: E402,F401
from .logging import P, T, debug, log_with_context, logger, setup_loki_logger, trace, trace_on  # noqa: E402,F401
from .neurons import *  # noqa: E402,F401,F403
from .schemas import Bucket, CommsGetResult  # noqa: E402,F401
from .dataset import DatasetLoader, SubsetLoader  # noqa: E402,F401
from .sharded_dataset import SharedShardedDataset, ShardedDatasetManager, SyntheticDataset, compute_shard_state  # noqa: E402,F401
from .sharded_sampler import EvalSampler, MinerSampler  # noqa: E402,F401
from .wandb_ops import initialize_wandb  # noqa: E402,F401
from .metrics import (DEFAULT_BUCKET as DEFAULT_DATABASE, DEFAULT_HOST, DEFAULT_ORG, DEFAULT_PORT, RUNTIME_ID,  # noqa: E402,F401
                      MetricsLogger, get_gpu_metrics, get_system_metrics)
from . import backends, metrics, model_factory, muon, profilers, wandb_ops  # noqa: E402,F401
