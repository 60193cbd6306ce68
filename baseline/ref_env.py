"""Import environment for running the UNMODIFIED reference (installed under ``baseline/_ref``)
on a box without network access.

Nothing in the reference's code is changed.  What this module does, in the way the reference's
own ``scripts/local_miner_test.py:93-161`` and ``tests/conftest.py:9-36`` do it:

* seeds the mock ``R2_*`` / ``DATASET_BINS_PATH`` variables that ``tplr.config`` requires at import;
* registers stand-in modules for third-party packages that are not installed offline
  (``bittensor``, ``boto3``/``botocore``/``aiobotocore``, ``influxdb_client``, ``logging_loki``,
  ``openskill``, ``zstandard``, ``multiprocessing_logging``) — none of them is on the compute path;
* the reference pins a *fork* of torchtitan whose LLaMA takes ``forward(tokens, labels)`` and has a
  ``tie_embeddings`` model argument; only upstream torchtitan is installed here, so the two
  fork-only API points are provided on top of the upstream classes (the model code that runs is
  upstream torchtitan's, i.e. the reference's dependency, not this repository's).
"""

from __future__ import annotations

import dataclasses
import os
import sys
import types
from pathlib import Path
from unittest.mock import MagicMock

REF_ROOT = Path(__file__).resolve().parent / "_ref"

_ENV = {
    "R2_GRADIENTS_ACCOUNT_ID": "mock-account", "R2_GRADIENTS_BUCKET_NAME": "mock-gradients",
    "R2_GRADIENTS_READ_ACCESS_KEY_ID": "mock-read", "R2_GRADIENTS_READ_SECRET_ACCESS_KEY": "mock-read-secret",
    "R2_GRADIENTS_WRITE_ACCESS_KEY_ID": "mock-write", "R2_GRADIENTS_WRITE_SECRET_ACCESS_KEY": "mock-write-secret",
    "R2_AGGREGATOR_ACCOUNT_ID": "mock-account", "R2_AGGREGATOR_BUCKET_NAME": "mock-aggregator",
    "R2_AGGREGATOR_READ_ACCESS_KEY_ID": "mock-read", "R2_AGGREGATOR_READ_SECRET_ACCESS_KEY": "mock-read-secret",
    "R2_AGGREGATOR_WRITE_ACCESS_KEY_ID": "mock-write", "R2_AGGREGATOR_WRITE_SECRET_ACCESS_KEY": "mock-write-secret",
    "R2_DATASET_ACCOUNT_ID": "mock-account", "R2_DATASET_BUCKET_NAME": "mock-dataset",
    "R2_DATASET_READ_ACCESS_KEY_ID": "mock-read", "R2_DATASET_READ_SECRET_ACCESS_KEY": "mock-read-secret",
    "DATASET_BINS_PATH": "/tmp/tplr-mock-bins",
}


class _Stub(types.ModuleType):
    """Module whose unknown attributes are MagicMocks (callable, attribute-rich, never on a hot path)."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        m = MagicMock(name=f"{self.__name__}.{name}")
        setattr(self, name, m)
        return m


def _stub(name: str, **attrs) -> types.ModuleType:
    parts = name.split(".")
    _STUB_ROOTS.add(parts[0])
    if not any(f is _StubFinder for f in sys.meta_path):
        sys.meta_path.append(_StubFinder)
    for i in range(1, len(parts) + 1):
        n = ".".join(parts[:i])
        if n not in sys.modules:
            mod = _Stub(n)
            mod.__path__ = []  # behaves as a package
            import importlib.machinery

            mod.__spec__ = importlib.machinery.ModuleSpec(n, None, is_package=True)
            sys.modules[n] = mod
            if i > 1:
                setattr(sys.modules[".".join(parts[:i - 1])], parts[i - 1], mod)
    mod = sys.modules[name]
    for k, v in attrs.items():
        setattr(mod, k, v)
    return mod


_STUB_ROOTS: set[str] = set()


class _StubFinder:
    """Resolves any submodule import below a stubbed package to another stand-in module."""

    @staticmethod
    def find_spec(fullname, path=None, target=None):
        import importlib.machinery

        if fullname.split(".")[0] in _STUB_ROOTS and fullname not in sys.modules:
            return importlib.machinery.ModuleSpec(fullname, _StubFinder, is_package=True)
        return None

    @staticmethod
    def create_module(spec):
        mod = _Stub(spec.name)
        mod.__path__ = []
        return mod

    @staticmethod
    def exec_module(module):
        return None


def _missing(name: str) -> bool:
    import importlib.util

    try:
        return importlib.util.find_spec(name) is None
    except (ImportError, ValueError):
        return True


def _stub_third_party() -> list[str]:
    stubbed = []
    exc = lambda n: type(n, (Exception,), {})  # noqa: E731
    if _missing("botocore"):
        _stub("botocore")
        _stub("botocore.config", Config=lambda **kw: types.SimpleNamespace(**kw))
        _stub("botocore.exceptions", ClientError=exc("ClientError"), ConnectionClosedError=exc("ConnectionClosedError"),
              EndpointConnectionError=exc("EndpointConnectionError"), NoCredentialsError=exc("NoCredentialsError"))
        stubbed.append("botocore")
    if _missing("boto3"):
        _stub("boto3")
        _stub("boto3.s3")
        _stub("boto3.s3.transfer")
        stubbed.append("boto3")
    if _missing("aiobotocore"):
        _stub("aiobotocore")
        _stub("aiobotocore.session")
        _stub("aiobotocore.client")
        _stub("aiobotocore.config")
        stubbed.append("aiobotocore")
    for name, subs in (("influxdb_client", ["client", "client.write_api", "client.exceptions", "rest"]),
                       ("logging_loki", []), ("openskill", ["models"]), ("zstandard", []),
                       ("multiprocessing_logging", []), ("bittensor", ["core", "core.chain_data", "core.subtensor",
                                                                       "utils", "utils.balance", "core.settings"])):
        if _missing(name):
            _stub(name)
            for s in subs:
                _stub(f"{name}.{s}")
            stubbed.append(name)
    if "bittensor" in stubbed:
        bt = sys.modules["bittensor"]

        class _Hotkey:
            ss58_address = "mock-hotkey"

        class _Wallet:
            def __init__(self, *a, **k):
                self.hotkey = _Hotkey()

            @staticmethod
            def add_args(_):
                return None

        class _Metagraph:
            def __init__(self):
                import torch

                self.hotkeys, self.uids, self.S, self.netuid, self.n = ["mock-hotkey"], [0], torch.tensor([1.0]), 3, 1

            def sync(self, *a, **k):
                return self

        class _Subtensor:
            block = 1000

            def __init__(self, *a, **k):
                pass

            @staticmethod
            def add_args(_):
                return None

            def metagraph(self, *_a, **_k):
                return _Metagraph()

        bt.wallet, bt.subtensor, bt.Wallet, bt.Subtensor = _Wallet, _Subtensor, _Wallet, _Subtensor
    return stubbed


def _torchtitan_fork_api() -> None:
    """``tie_embeddings`` model argument and ``forward(tokens, labels)`` on the upstream classes."""
    import torch
    import torchtitan.models.llama3 as l3

    base_args = l3.TransformerModelArgs
    if "tie_embeddings" not in {f.name for f in dataclasses.fields(base_args)}:
        @dataclasses.dataclass
        class TransformerModelArgs(base_args):  # type: ignore[misc,valid-type]
            tie_embeddings: bool = False

        l3.TransformerModelArgs = TransformerModelArgs
        for modname in ("torchtitan.models.llama3.model.args", "torchtitan.models.llama3.model"):
            mod = sys.modules.get(modname)
            if mod is not None and hasattr(mod, "TransformerModelArgs"):
                mod.TransformerModelArgs = TransformerModelArgs
    base_model = l3.Transformer
    import inspect

    if "labels" not in inspect.signature(base_model.forward).parameters:
        class Transformer(base_model):  # type: ignore[misc,valid-type]
            def __init__(self, model_args):
                super().__init__(model_args)
                if getattr(model_args, "tie_embeddings", False) and self.output is not None:
                    self.output.weight = self.tok_embeddings.weight

            def forward(self, tokens: torch.Tensor, labels: torch.Tensor | None = None, **kw):
                return super().forward(tokens)

        Transformer.__name__ = base_model.__name__
        l3.Transformer = Transformer


def prepare(stub: bool = True) -> dict:
    """Make ``import tplr`` / ``import neurons`` resolve to the installed reference. Returns a report."""
    if not (REF_ROOT / "tplr").is_dir():
        raise FileNotFoundError(f"reference is not installed under {REF_ROOT}")
    for k, v in _ENV.items():
        os.environ.setdefault(k, v)
    os.makedirs(os.environ["DATASET_BINS_PATH"], exist_ok=True)
    _torchtitan_fork_api()          # imports torchtitan (and its real dependencies) before any stand-in exists
    stubbed = _stub_third_party() if stub else []
    p = str(REF_ROOT)
    if p in sys.path:
        sys.path.remove(p)
    sys.path.insert(0, p)
    for name in [n for n in sys.modules if n == "tplr" or n.startswith("tplr.") or n == "neurons" or n.startswith("neurons.")]:
        del sys.modules[name]
    return {"ref_root": p, "stubbed": stubbed}
