"""The flat public namespace (the reference's ``tplr.*``, src/tplr/__init__.py:22-40) and the ``tplr`` alias package."""

import inspect

import templar_b200

# name -> parameters the reference's callers pass by keyword (a subset of each signature)
SURFACE = {
    "Comms": ["wallet", "save_location", "key_prefix", "config", "hparams", "uid"],
    "ChainManager": [],
    "DCPCheckpointer": ["comms", "uid", "version", "repo_root"],
    "MinerSampler": ["dataset", "uid", "window", "steps_per_window", "micro_bs", "batch_size", "target_batch_size", "rank", "world_size"],
    "EvalSampler": ["dataset", "uid", "window", "steps_per_window", "micro_bs", "batch_size", "validation_bs", "rank", "world_size"],
    "SharedShardedDataset": ["shard_index", "sequence_length", "rank", "world_size"],
    "ChunkingTransformer": ["model", "target_chunk"],
    "TopKCompressor": ["use_quantization", "quantization_bins", "quantization_range"],
    "MetricsLogger": ["prefix", "uid", "config", "role", "group", "job_type"],
    "prepare_gradient_dict": ["miner", "step_window", "null_round"],
    "outer_step": ["model", "optimizer", "gather_result", "transformer", "compressor", "xshapes", "totalks", "device",
                   "is_master", "world_size", "use_dct", "wandb_run", "global_step"],
    "update_peers": ["instance", "window", "peer_start"],
    "load_checkpoint_with_fallback": ["instance"],
    "handle_checkpoint_catchup": ["instance"],
    "catchup_with_aggregation_server": ["instance", "checkpoint_current_window"],
    "compare_model_with_debug_dict": ["model", "debug_dict", "learning_rate", "param_avg_change", "min_step_size", "index_range"],
    "check_uid_index_overlap": ["neuron", "gather_result", "window", "overlap_threshold"],
    "determine_slash_egregiousness": [], "instantiate_slashing_multiplier": [],
    "pack_12bit_indices": ["indices"], "unpack_12bit_indices": ["packed", "values_shape"],
    "load_hparams": ["hparams_dir", "use_local_run_hparams"],
    "initialize_wandb": [], "Bucket": [], "CommsGetResult": [],
    "logger": None, "T": None, "P": None, "log_with_context": None, "setup_loki_logger": None,
    "muon": None, "distributed": None, "compress": None,
}


def test_flat_namespace_has_the_reference_surface():
    for name, params in SURFACE.items():
        assert hasattr(templar_b200, name), name
        if params:
            obj = getattr(templar_b200, name)
            sig = inspect.signature(obj.__init__ if inspect.isclass(obj) else obj)
            missing = [p for p in params if p not in sig.parameters]
            assert not missing, (name, missing)
    assert templar_b200.muon.Muon and templar_b200.muon.SingleDeviceMuonWithAuxAdam
    assert templar_b200.distributed.dist_helper is not None


def test_tplr_is_the_same_package_under_the_reference_name():
    import tplr
    import tplr.compress
    import tplr.neurons
    from tplr.compress import TopKCompressor
    from tplr.muon import Muon
    import tplr.distributed as d

    assert tplr.__version__ == templar_b200.__version__
    assert tplr.compress is templar_b200.compress and tplr.neurons is templar_b200.neurons
    assert tplr.Comms is templar_b200.Comms and TopKCompressor is templar_b200.compress.TopKCompressor
    assert Muon is templar_b200.muon.Muon and d.dist_helper is templar_b200.distributed.dist_helper
    assert tplr.initialize_wandb is templar_b200.wandb_ops.initialize_wandb
    assert tplr.MetricsLogger is templar_b200.metrics.MetricsLogger


def test_every_public_name_of_the_reference_package_root_resolves():
    """The reference's root star-imports chain, comms, compress, dataset, neurons, hparams, logging, schemas and
    metrics (src/tplr/__init__.py:26-35).  Their public top-level names, listed here from those files: a caller's
    ``tplr.<name>`` keeps resolving.  Omitted on purpose: the InfluxDB fallback token and write-options class of the
    reference's metrics module (this package takes the token from the environment only)."""
    names = """
      ChainManager Comms CF_REGION_NAME LOCAL_TMP_DIR PEERS_FILE_PREFIX CPU_COUNT CPU_MAX_CONNECTIONS SAFE_BUCKET_RE SAFE_KEY_RE
      ShapeT Shape4D TotK IdxT QuantParamsT ValT pack_12bit_indices unpack_12bit_indices ChunkingTransformer TopKCompressor
      DatasetLoader SubsetLoader NeuronT prepare_gradient_dict outer_step update_peers load_checkpoint_with_fallback
      handle_checkpoint_catchup catchup_with_aggregation_server compare_model_with_debug_dict check_uid_index_overlap
      determine_slash_egregiousness instantiate_slashing_multiplier DEFAULT_HPARAMS create_namespace load_hparams
      logger T P debug trace log_with_context setup_loki_logger Bucket CommsGetResult MetricsLogger RUNTIME_ID DEFAULT_HOST
      DEFAULT_PORT DEFAULT_DATABASE DEFAULT_ORG get_gpu_metrics get_system_metrics initialize_wandb SharedShardedDataset
      EvalSampler MinerSampler DCPCheckpointer muon distributed
    """.split()
    import tplr

    missing = [n for n in names if not hasattr(templar_b200, n) or not hasattr(tplr, n)]
    assert not missing, missing
    assert templar_b200.SAFE_KEY_RE.match("checkpoints/2.1.28/5/__0_0.distcp") and not templar_b200.SAFE_BUCKET_RE.match("a/b")
    ns = templar_b200.create_namespace({"topk_compression": 7})
    assert ns.topk_compression == 7 and hasattr(ns, "blocks_per_window")


def test_methods_and_module_names_callers_of_the_reference_use():
    from templar_b200 import profilers
    from templar_b200.muon import muon as muon_mod

    for name in ("upload_large_file", "download_large_file", "s3_get_object_range", "s3_get_object_size", "s3_put_object",
                 "s3_get_object", "gather", "gather_with_reserve", "get_with_retry", "put", "get", "post_peer_list",
                 "post_start_window", "get_peer_list", "get_start_window", "check_compressed_indices", "is_miner_active",
                 "track_active_peers", "get_debug_dict", "weighted_random_sample_no_replacement", "cleanup_local_data",
                 "cleanup_s3_data", "gradient_timestamp", "get_own_bucket", "get_base_url", "delete_local_directory",
                 "start_background_tasks"):
        assert callable(getattr(templar_b200.Comms, name, None)), name
    assert callable(templar_b200.ChainManager.decode_metadata)
    for name in ("apply_momentum", "apply_scaling", "adam_update", "zeropower_via_newtonschulz5",
                 "zeropower_via_newtonschulz5_optimized", "Muon", "SingleDeviceMuonWithAuxAdam"):
        assert hasattr(muon_mod, name), name
    for name in ("ENABLE_PROFILERS", "ENABLE_TIMER_PROFILER", "ENABLE_SHARD_PROFILER", "get_timer_profiler", "get_profiler"):
        assert hasattr(profilers, name), name
    import torch
    g, m = torch.ones(4, 2), torch.zeros(4, 2)
    u = templar_b200.muon.apply_momentum(g, m, 0.5, nesterov=True)
    assert torch.allclose(m, torch.full((4, 2), 0.5)) and torch.allclose(u, torch.full((4, 2), 0.75))
    assert torch.allclose(templar_b200.muon.apply_scaling(torch.ones(4, 2)), torch.full((4, 2), 2 ** 0.5))
    assert torch.allclose(templar_b200.muon.apply_scaling(torch.ones(4, 2), rms_scale=True), torch.full((4, 2), 0.4))
