"""Model construction per role, parallel-dimension validation and HF export.

Same entry points as the reference's src/tplr/model_factory.py:60-739, built on this
framework's own LLaMA (:mod:`templar_b200.models.llama`) and sharding engine instead of
torchtitan + FSDP2:

* ``get_titan_model_args``    hparams -> :class:`ModelArgs` (preset sizes or custom geometry, the FFN
  width taken verbatim from ``intermediate_size``);
* ``create_parallel_dims``    role rules: evaluator ``dp_shard = min(8, world)``, validator ``dp_shard = 4``
  (both with replication over the rest), miner from ``hparams.torchtitan`` with the reference's
  validation errors (:func:`create_parallel_dims` raises the same messages);
* ``create_job_config``       the execution options the engine honours (compute dtype, fp32 reduction,
  activation checkpointing, CPU offload of optimizer state);
* ``create_meta_model`` / ``initialize_torchtitan_model`` / ``initialize_weights_inplace``
  deterministic seed-42 initialisation, identical on every rank without a broadcast (every rank
  draws the same stream), so start-up needs no rank-0 scatter of the full state dict;
* ``convert_titan_to_hf``     state-dict conversion to the HuggingFace LLaMA layout, including the
  interleaved -> half-rotation permutation of the q/k projection rows.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Any, Literal

import torch
import torch.nn as nn

from .logging import logger
from .models.llama import PRESETS, LlamaModel, ModelArgs

TransformerModelArgs = ModelArgs       # name used by callers written against the reference
llama3_configs = {k: v for k, v in PRESETS.items() if k in ("8B", "70B")}


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    world_size: int = 1

    def __post_init__(self):
        if self.dp_shard == -1:
            self.dp_shard = self.world_size // (self.dp_replicate * self.tp * self.pp * self.cp)
        prod = self.dp_replicate * self.dp_shard * self.tp * self.pp * self.cp
        if prod != self.world_size and self.world_size % max(prod, 1) != 0:
            raise ValueError(f"Invalid parallel dims: {prod} does not divide world_size {self.world_size}")

    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate > 1 or self.dp_shard > 1

    @property
    def dp_shard_enabled(self) -> bool:
        return self.dp_shard > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    def mesh_shape(self) -> dict[str, int]:
        return {k: v for k, v in (("pp", self.pp), ("dp_replicate", self.dp_replicate), ("dp_shard", self.dp_shard),
                                  ("cp", self.cp), ("tp", self.tp)) if v > 1}


@dataclass
class JobConfig:
    seq_len: int = 2048
    compile: bool = False                       # accepted for compatibility; kernels are hand-written
    enable_cpu_offload: bool = False
    mixed_precision_param: str = "bfloat16"
    mixed_precision_reduce: str = "float32"     # gradients are always reduced in fp32
    enable_async_tensor_parallel: bool = False
    disable_loss_parallel: bool = True
    fsdp_reshard_after_forward: str = "default"
    enable_compiled_autograd: bool = False
    float8_recipe_name: str | None = None
    activation_checkpoint_mode: str = "selective"
    selective_ac_option: str = "op"
    converters: list = field(default_factory=list)


def get_titan_model_args(hparams: SimpleNamespace) -> ModelArgs:
    size = hparams.model_size
    seq = hparams.sequence_length
    vocab = hparams.tokenizer.vocab_size if hasattr(hparams, "tokenizer") else hparams.model_config.vocab_size
    tt = getattr(hparams, "torchtitan", SimpleNamespace())
    tie = getattr(tt, "tie_embeddings", True)
    if size in llama3_configs:
        base = llama3_configs[size]
        return ModelArgs(**{**base.__dict__, "max_seq_len": seq, "vocab_size": vocab, "tie_embeddings": tie})
    mc = hparams.model_config
    return ModelArgs(dim=mc.hidden_size, n_layers=mc.num_hidden_layers, n_heads=mc.num_attention_heads,
                     n_kv_heads=getattr(mc, "num_key_value_heads", mc.num_attention_heads), vocab_size=vocab,
                     intermediate_size=mc.intermediate_size, multiple_of=256,
                     ffn_dim_multiplier=mc.intermediate_size / max(int(8 * mc.hidden_size / 3), 1),
                     norm_eps=getattr(mc, "rms_norm_eps", 1e-5), rope_theta=getattr(mc, "rope_theta", 10000.0),
                     max_seq_len=seq, tie_embeddings=tie)


def create_job_config(hparams: SimpleNamespace, role: Literal["miner", "validator", "evaluator"] = "miner") -> JobConfig:
    tt = getattr(hparams, "torchtitan", SimpleNamespace())
    mp = "bfloat16" if getattr(tt, "mixed_precision_param", "float32") == "bfloat16" else "float32"
    offload = False
    if role == "evaluator":
        mp = "float32"
    elif role == "miner":
        offload = getattr(tt, "enable_cpu_offload", False)
    ac = getattr(tt, "activation_checkpoint", None)
    ac = ac if isinstance(ac, dict) else {}
    return JobConfig(seq_len=hparams.sequence_length, compile=getattr(tt, "compile", False), enable_cpu_offload=offload,
                     mixed_precision_param=mp, mixed_precision_reduce="float32",
                     enable_async_tensor_parallel=getattr(tt, "enable_async_tensor_parallel", False),
                     disable_loss_parallel=getattr(tt, "disable_loss_parallel", True),
                     fsdp_reshard_after_forward=getattr(tt, "fsdp_reshard_after_forward", "default"),
                     enable_compiled_autograd=getattr(tt, "enable_compiled_autograd", False),
                     float8_recipe_name=getattr(tt, "float8_recipe_name", None),
                     activation_checkpoint_mode=ac.get("mode", "selective"), selective_ac_option=ac.get("option", "op"),
                     converters=list(getattr(tt, "converters", [])))


def create_parallel_dims(world_size: int, hparams: SimpleNamespace,
                         role: Literal["miner", "validator", "evaluator"] = "miner") -> ParallelDims:
    if world_size <= 0:
        world_size = 1
    if role in ("evaluator", "validator"):
        dp_shard = max(1, min(8, world_size)) if role == "evaluator" else 4
        if world_size % dp_shard != 0:
            raise ValueError(f"World size ({world_size}) must be divisible by dp_shard degree ({dp_shard})")
        return ParallelDims(dp_replicate=world_size // dp_shard, dp_shard=dp_shard, world_size=world_size)
    tt = getattr(hparams, "torchtitan", SimpleNamespace())
    deg = {k: getattr(tt, k, 1) for k in ("dp_replicate", "dp_shard", "tp_degree", "pp_degree", "cp_degree")}
    for k, v in deg.items():
        if v == 0:
            raise ValueError(f"{k} cannot be zero.")
    deg = {k: int(v) for k, v in deg.items()}
    if deg["dp_shard"] == -1:       # "use whatever is left of the world": an addition to the reference's rules
        rest = deg["dp_replicate"] * deg["tp_degree"] * deg["pp_degree"] * deg["cp_degree"]
        deg["dp_shard"] = max(world_size // max(rest, 1), 1)
    if deg["dp_replicate"] > 1 and deg["dp_shard"] > 1:
        raise ValueError("Specify either torchtitan.dp_replicate or torchtitan.dp_shard, but not both.")
    if deg["dp_replicate"] > 1 and (deg["tp_degree"] > 1 or deg["pp_degree"] > 1 or deg["cp_degree"] > 1):
        raise ValueError("dp_replicate can only be used when tp/pp/cp are all 1.")
    total = deg["dp_replicate"] * deg["dp_shard"] * deg["tp_degree"] * deg["pp_degree"] * deg["cp_degree"]
    if total == 0:
        raise ValueError("Product of parallel degrees cannot be zero.")
    if world_size % total != 0:
        raise ValueError(f"world_size ({world_size}) must be divisible by the product of all parallel degrees "
                         f"({deg['dp_replicate']}x{deg['dp_shard']}x{deg['tp_degree']}x{deg['pp_degree']}x{deg['cp_degree']} = {total}).")
    return ParallelDims(dp_replicate=deg["dp_replicate"], dp_shard=deg["dp_shard"], tp=deg["tp_degree"],
                        pp=deg["pp_degree"], cp=deg["cp_degree"], ep=1, world_size=world_size)


def _compute_dtype(job: JobConfig, device) -> torch.dtype:
    if torch.device(device).type != "cuda":
        return torch.float32
    return torch.bfloat16 if job.mixed_precision_param == "bfloat16" else torch.float32


def create_meta_model(hparams: SimpleNamespace, role: Literal["miner", "validator", "evaluator"] = "miner",
                      world_size: int = 1) -> nn.Module:
    """Structure only (meta device): used when a checkpoint will provide the weights."""
    args = get_titan_model_args(hparams)
    pdims = create_parallel_dims(world_size, hparams, role)
    job = create_job_config(hparams, role)
    with torch.device("meta"):
        model = LlamaModel(args)
    model.parallel_dims, model.job_config = pdims, job
    # torchtitan.activation_checkpoint of the hparams: {"mode": "none" | "full" | "selective", "option": "op" | "<N>"}
    # (reference src/tplr/model_factory.py:195-204)
    mode = str(job.activation_checkpoint_mode or "none").lower()
    if mode not in ("none", "full", "selective"):
        raise ValueError(f"activation_checkpoint.mode must be none, full or selective, got {mode!r}")
    model.activation_checkpointing = mode
    model.ac_option = str(job.selective_ac_option)
    return model


def materialize(model: LlamaModel, device) -> LlamaModel:
    """``to_empty`` plus re-creation of the rotary buffer (meta tensors carry no values)."""
    model.to_empty(device=device)
    model.freqs_cis = model._freqs_cis().to(device)
    model._rope_cache.clear()
    return model


def initialize_weights_inplace(model: nn.Module, hparams: SimpleNamespace | None = None, world_size: int = 1,
                               seed: int = 42) -> None:
    """Seeded initialisation on the model's own device.  Every rank generates the same values
    (host generator, then copied), which replaces the reference's rank-0 init + broadcast."""
    dev = next(model.parameters()).device
    args = model.args
    ref = LlamaModel(args)
    torch.manual_seed(seed)
    ref.init_weights(seed)
    sd = ref.state_dict()
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(sd[name].to(device=dev, dtype=p.dtype))
        model.freqs_cis = sd["freqs_cis"].to(dev)
    engine = getattr(model, "_window_engine", None)
    if engine is not None:
        engine.load_full_state_dict({k: v for k, v in sd.items()})


def initialize_torchtitan_model(hparams: SimpleNamespace, role: Literal["miner", "validator", "evaluator"] = "miner",
                                device: str = "cuda", world_size: int = 1) -> nn.Module:
    model = create_meta_model(hparams, role, world_size)
    materialize(model, device)
    job = model.job_config
    dt = _compute_dtype(job, device)
    if dt != torch.float32:
        fc = model.freqs_cis
        model.to(dt)
        model.freqs_cis = fc
    initialize_weights_inplace(model, hparams, world_size)
    logger.info(f"[Model Factory] Initialized {role} model on {device} ({model.args.num_params() / 1e6:.1f} M params, {dt})")
    return model


# --------------------------------------------------------------------------------------- #
# HuggingFace export
# --------------------------------------------------------------------------------------- #
_HF_MAP = {"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight",
           "output.weight": "lm_head.weight"}
_HF_LAYER = {"attention.wq.weight": "self_attn.q_proj.weight", "attention.wk.weight": "self_attn.k_proj.weight",
             "attention.wv.weight": "self_attn.v_proj.weight", "attention.wo.weight": "self_attn.o_proj.weight",
             "feed_forward.w1.weight": "mlp.gate_proj.weight", "feed_forward.w3.weight": "mlp.up_proj.weight",
             "feed_forward.w2.weight": "mlp.down_proj.weight", "attention_norm.weight": "input_layernorm.weight",
             "ffn_norm.weight": "post_attention_layernorm.weight"}


def _interleaved_to_half_rotation(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Rows of a q/k projection: (head, pair, 2) order -> (head, 2, pair) order, the layout of
    HF's rotate-half RoPE."""
    rows, cols = w.shape
    hd = rows // n_heads
    return w.view(n_heads, hd // 2, 2, cols).transpose(1, 2).reshape(rows, cols)


def titan_to_hf_state_dict(sd: dict, args: ModelArgs) -> dict:
    out = {}
    for k, v in sd.items():
        if "freqs_cis" in k:
            continue
        k = k.replace("_orig_mod.", "").replace("module.", "")
        if k in _HF_MAP:
            out[_HF_MAP[k]] = v
            continue
        if k.startswith("layers."):
            _, idx, rest = k.split(".", 2)
            name = _HF_LAYER.get(rest)
            if name is None:
                continue
            if rest == "attention.wq.weight":
                v = _interleaved_to_half_rotation(v, args.n_heads)
            elif rest == "attention.wk.weight":
                v = _interleaved_to_half_rotation(v, args.kv_heads)
            out[f"model.layers.{idx}.{name}"] = v
    if args.tie_embeddings and "lm_head.weight" not in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out


def _hf_config_dict(args: ModelArgs, hparams: SimpleNamespace) -> dict:
    mc = getattr(hparams, "model_config", SimpleNamespace())
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=args.vocab_size,
                hidden_size=args.dim, intermediate_size=args.ffn_hidden, num_hidden_layers=args.n_layers,
                num_attention_heads=args.n_heads, num_key_value_heads=args.kv_heads,
                hidden_act=getattr(mc, "hidden_act", "silu"), max_position_embeddings=hparams.sequence_length,
                initializer_range=getattr(mc, "initializer_range", 0.02), rms_norm_eps=args.norm_eps, use_cache=False,
                rope_theta=args.rope_theta, rope_scaling=None, attention_bias=False, attention_dropout=0.0,
                pretraining_tp=1, tie_word_embeddings=False, torch_dtype="float32")


def convert_titan_to_hf(titan_model: nn.Module, hparams: SimpleNamespace, save_path: str | None = None,
                        model_args: dict[str, Any] | None = None, is_master: bool = False):
    """Gathers the full fp32 state (all ranks participate), converts it on the master rank and,
    when ``save_path`` is given, writes ``config.json`` + ``pytorch_model.bin`` (or a
    ``save_pretrained`` directory when transformers can build the model)."""
    from .dcp_checkpoint import model_state_dict

    inner = titan_model
    while hasattr(inner, "module"):
        inner = inner.module
    sd = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in model_state_dict(inner).items()}
    if not is_master:
        return None
    args = inner.args
    hf_sd = titan_to_hf_state_dict(sd, args)
    cfg = model_args or _hf_config_dict(args, hparams)
    hf_model = None
    try:
        from transformers import LlamaConfig, LlamaForCausalLM

        hf_model = LlamaForCausalLM(LlamaConfig(**{k: v for k, v in cfg.items() if k not in ("architectures", "model_type", "torch_dtype")}))
        hf_model.load_state_dict({k: v.float() for k, v in hf_sd.items()}, strict=True)
    except Exception as e:  # noqa: BLE001
        logger.warning(f"transformers model could not be built ({e}); writing raw state dict")
        hf_model = None
    if save_path:
        os.makedirs(save_path, exist_ok=True)
        if hf_model is not None:
            hf_model.save_pretrained(save_path)
        else:
            with open(os.path.join(save_path, "config.json"), "w") as f:
                json.dump(cfg, f, indent=2)
            torch.save(hf_sd, os.path.join(save_path, "pytorch_model.bin"))
    return hf_model if hf_model is not None else hf_sd


# --------------------------------------------------------------------------------------- #
# Deterministic-initialisation check
# --------------------------------------------------------------------------------------- #
def model_fingerprint(model: nn.Module) -> str:
    """MD5 over the bytes of every parameter in ``named_parameters`` order (fp32 view), preceded by its name."""
    import hashlib

    h = hashlib.md5()
    for name, p in model.named_parameters():
        h.update(name.encode())
        h.update(p.detach().float().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()


def check_init(hparams: SimpleNamespace, role: str = "miner", device: str = "cpu", builds: int = 2) -> dict:
    """Build the model ``builds`` times and compare the parameters: every node of the network must start from the
    same weights, so two builds with the same hparams have to agree to the last bit (the check of the reference's
    scripts/test_init.py).  Returns the fingerprints and the names of tensors that differ from the first build."""
    first, prints, differing = None, [], []
    for _ in range(builds):
        m = initialize_torchtitan_model(hparams, role=role, device=device, world_size=1)
        prints.append(model_fingerprint(m))
        sd = {n: p.detach().float().cpu() for n, p in m.named_parameters()}
        if first is None:
            first = sd
        else:
            differing += [n for n in first if n not in sd or not torch.equal(first[n], sd[n])]
        del m
    return {"fingerprints": prints, "identical": len(set(prints)) == 1 and not differing, "differing": sorted(set(differing))}


if __name__ == "__main__":          # python -m templar_b200.model_factory [--hparams-dir hparams] [--device cpu]
    import argparse

    from .hparams import load_hparams

    _ap = argparse.ArgumentParser(description="check that the model initialisation is deterministic")
    _ap.add_argument("--hparams-dir", default="hparams")
    _ap.add_argument("--role", default="miner", choices=["miner", "validator", "evaluator"])
    _ap.add_argument("--device", default="cpu")
    _a = _ap.parse_args()
    _rep = check_init(load_hparams(_a.hparams_dir), _a.role, _a.device)
    print(json.dumps(_rep))
    raise SystemExit(0 if _rep["identical"] else 1)
