"""Hyper-parameter loading.

Merge order (reference src/tplr/hparams.py:126-207): built-in defaults -> ``hparams/hparams.json``
-> ``hparams/<model_size>.json`` (skipped when ``model_size`` names a built-in architecture preset)
-> ``hparams/hparams-local-run.json`` when requested.  The result is a ``SimpleNamespace`` with the
``torchtitan`` sub-dict exposed as its own namespace, a tokenizer whose pad token is its eos token,
and a ``model_config`` with the LLaMA geometry.  Offline there is no tokenizer download: when the
named tokenizer is not in the local HF cache a :class:`SyntheticTokenizer` with the model's
vocabulary size stands in.
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from types import SimpleNamespace

from .logging import logger

DEFAULT_HPARAMS = {
    "spec_version": 5, "project": "templar",
    "sequence_length": 1024, "pages_per_window": 2, "batch_size": 8, "learning_rate": 0.001,
    "blocks_per_window": 2, "windows_per_weights": 10,
    "momentum_decay": 0.999, "topk_compression": 32, "target_chunk": 64, "scores_alpha": 0.001,
    "tokenizer_name": "huggyllama/llama-7b", "hidden_size": 4096, "num_hidden_layers": 32,
    "num_attention_heads": 32, "intermediate_size": 11008, "num_key_value_heads": 32,
    "activation_function": "silu", "max_position_embeddings": 2048,
    "bucket_name": "your-default-bucket-name",
    "warmup_steps": 250, "alpha_f": 0.1, "t_max": 20000,
    "outer_steps_per_shard": 455,
}

# architecture presets that need no <model_size>.json (public llama3 tables)
PRESET_MODEL_SIZES = {"8B", "70B", "405B"}
KNOWN_VOCABS = {"togethercomputer/LLaMA-2-7B-32K": 32000, "huggyllama/llama-7b": 32000,
                "google/gemma-3-270m": 262144, "meta-llama/Llama-3.1-8B": 128256}


class SyntheticTokenizer:
    """Stand-in with the attributes the framework reads: vocab size and pad/eos/bos ids."""

    def __init__(self, vocab_size: int = 32000, name: str = "synthetic"):
        self.vocab_size = int(vocab_size)
        self.name_or_path = name
        self.bos_token_id, self.eos_token_id = 1, 2
        self.pad_token_id = self.eos_token_id
        self.eos_token = self.pad_token = "</s>"

    def __len__(self):
        return self.vocab_size

    def encode(self, text: str, **_) -> list[int]:
        return [3 + (b % (self.vocab_size - 3)) for b in text.encode("utf-8")]

    def decode(self, ids, **_) -> str:
        return bytes((int(i) - 3) % 256 for i in ids).decode("utf-8", errors="replace")


def load_tokenizer(name: str, vocab_hint: int | None = None):
    if os.environ.get("TPLR_SYNTHETIC_TOKENIZER", "0") != "1":
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(name, local_files_only=os.environ.get("HF_HUB_OFFLINE", "1") == "1",
                                                token=os.getenv("HF_TOKEN") or os.getenv("HUGGING_FACE_HUB_TOKEN"))
            tok.pad_token = tok.eos_token
            return tok
        except Exception as e:  # noqa: BLE001
            logger.debug(f"tokenizer {name} unavailable locally ({type(e).__name__}); using a synthetic one")
    return SyntheticTokenizer(vocab_hint or KNOWN_VOCABS.get(name, 32000), name)


def create_namespace(hparams: dict) -> SimpleNamespace:
    full = dict(DEFAULT_HPARAMS)
    full.update(hparams)
    ns = SimpleNamespace(**full)
    if isinstance(full.get("torchtitan"), dict):
        ns.torchtitan = SimpleNamespace(**full["torchtitan"])
    ns.tokenizer = load_tokenizer(ns.tokenizer_name, full.get("vocab_size"))
    ns.model_config = SimpleNamespace(
        vocab_size=full.get("vocab_size") or ns.tokenizer.vocab_size, hidden_size=ns.hidden_size,
        num_hidden_layers=ns.num_hidden_layers, num_attention_heads=ns.num_attention_heads,
        intermediate_size=ns.intermediate_size, num_key_value_heads=ns.num_key_value_heads,
        activation_function=ns.activation_function, max_position_embeddings=ns.max_position_embeddings,
        rms_norm_eps=full.get("rms_norm_eps", 1e-5), rope_theta=full.get("rope_theta", 10000.0))
    return ns


def _read(path: Path) -> dict:
    with open(path) as f:
        return json.load(f)


def load_hparams(hparams_dir: str = "hparams", use_local_run_hparams: bool = False) -> SimpleNamespace:
    root = Path(hparams_dir)
    base = root / "hparams.json"
    hp = dict(DEFAULT_HPARAMS)
    try:
        hp.update(_read(base))
    except FileNotFoundError:
        logger.error(f"CRITICAL: Base config file not found at {base}")
        raise
    size = hp.get("model_size")
    if not size:
        raise ValueError(f"CRITICAL: 'model_size' must be defined in {base}")
    if size not in PRESET_MODEL_SIZES:
        try:
            hp.update(_read(root / f"{size}.json"))
        except FileNotFoundError:
            raise ValueError(f"Could not find hparams for model_size '{size}'") from None
    if use_local_run_hparams:
        local = root / "hparams-local-run.json"
        if local.exists():
            hp.update(_read(local))
        else:
            logger.warning(f"Local run specified but {local} not found.")
    logger.info(f"Final project: '{hp.get('project')}', Model size: '{hp.get('model_size')}'")
    return create_namespace(hp)
