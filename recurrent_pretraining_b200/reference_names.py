"""Where a symbol of the reference lives in this package.

Scripts written against the reference import names such as ``recpre.huggingface_dataset.ParquetStreamPure`` or
``recpre.monitor.track_gradient_metrics``.  This package is laid out differently and names things after what they do
here; the table below maps every public reference symbol that has a counterpart to that counterpart, so a port of a
script is a lookup rather than a search:

    from recurrent_pretraining_b200 import reference_names as ref
    ParquetStreamPure = ref.ParquetStreamPure                       # by bare name (unique ones)
    cls = ref.resolve("recpre.huggingface_dataset.ParquetStreamPure")  # or by the reference's dotted path

Entries are ``"<reference dotted path>": "<module under this package>:<attribute>"`` and are imported lazily.  A
counterpart keeps the reference's behaviour and argument names unless its docstring says otherwise; kernels and
private helpers of the reference (its Triton kernels, the Lightning wrappers, the Inductor patches) have no entry:
their work is done inside the CUDA library or is not needed.
"""
from __future__ import annotations

import importlib
from typing import Any

_PKG = __name__.rsplit(".", 1)[0]

REFERENCE_NAMES: dict[str, str] = {
    # ---- train.py ------------------------------------------------------------------------------------------------
    "train.set_torch_flags": "runtime.trainer:set_torch_flags",
    "train.setup_fabric": "runtime.trainer:setup_fabric",
    "train.startup": "runtime.trainer:startup",
    "train.validate": "runtime.trainer:validate",
    "train.train": "runtime.trainer:train",
    "train.main": "runtime.trainer:main",
    "train.create_dataloader": "runtime.trainer:create_dataloader",
    "train.derive_precision": "runtime.trainer:derive_precision",
    "train.get_attention_mask": "runtime.trainer:get_attention_mask",
    "train.get_lr": "optim.schedules:get_lr",
    "train.get_batch_size": "optim.schedules:get_batch_size",
    "train.load_checkpoint": "runtime.checkpoint:load_checkpoint",
    "train.maybe_save_checkpoint": "runtime.trainer:maybe_save",
    "train.warmup_or_early_fail_allreduce": "runtime.trainer:warmup_or_early_fail_allreduce",
    "train._get_time_from_slurm": "runtime.trainer:slurm_seconds_left",
    "train.train_step": "runtime.engine:TrainEngine",                  # TrainEngine.train_step
    # ---- recpre/settings.py, config_dynamic.py, model_registry.py ---------------------------------------------------
    "recpre.settings.HuggingfaceConfig": "settings:HuggingfaceConfig",
    "recpre.settings.DataEntry": "settings:DataEntry",
    "recpre.settings.GoldfishConfig": "settings:GoldfishConfig",
    "recpre.settings.FabricConfig": "settings:FabricConfig",
    "recpre.settings.CLISettings": "settings:CLISettings",
    "recpre.config_dynamic.RoPESettings": "config:RoPESettings",
    "recpre.config_dynamic.Config": "config:ModelConfig",
    "recpre.config_dynamic.GPTConfig": "config:ModelConfig",
    "recpre.config_dynamic.RecurrentConfig": "config:ModelConfig",
    "recpre.config_dynamic.Linear": "models.blocks:Linear",
    "recpre.config_dynamic.Relu2": "models.blocks:Relu2",
    "recpre.model_registry.name_to_config": "registry:lookup",
    "recpre.raven_config_minimal.RavenConfig": "models.hf_config:RavenConfig",
    # ---- recpre/model_dynamic.py --------------------------------------------------------------------------------------
    "recpre.model_dynamic.RecurrentGPT": "models.recurrent:RecurrentGPT",
    "recpre.model_dynamic.GPT": "models.recurrent:GPT",
    "recpre.model_dynamic.CausalSelfAttention": "models.blocks:CausalSelfAttention",
    "recpre.model_dynamic.DiffSelfAttention": "models.variants:DiffSelfAttention",
    "recpre.model_dynamic.SimplifiedDiffSelfAttention": "models.variants:SimplifiedDiffSelfAttention",
    "recpre.model_dynamic.PositionalAttention": "models.variants:PositionalAttention",
    "recpre.model_dynamic.OPSelfAttention": "models.variants:OPSelfAttention",
    "recpre.model_dynamic.BaseMLP": "models.blocks:BaseMLP",
    "recpre.model_dynamic.GatedMLP": "models.blocks:GatedMLP",
    "recpre.model_dynamic.GatedMLPSeparated": "models.variants:GatedMLPSeparated",
    "recpre.model_dynamic.HalfGateMLP": "models.variants:HalfGateMLP",
    "recpre.model_dynamic.TimestepEmbedder": "models.variants:TimestepEmbedder",
    "recpre.model_dynamic.TransformerScaledPreNormBlock": "models.blocks:TransformerScaledPreNormBlock",
    "recpre.model_dynamic.TransformerPreNormBlock": "models.blocks:TransformerPreNormBlock",
    "recpre.model_dynamic.TransformerPostNormBlock": "models.blocks:TransformerPostNormBlock",
    "recpre.model_dynamic.ScaledTransformerPostNormBlock": "models.blocks:ScaledTransformerPostNormBlock",
    "recpre.model_dynamic.OPTransformerBlock": "models.variants:OPTransformerBlock",
    "recpre.model_dynamic.SwinScaledBlock": "models.variants:SwinScaledBlock",
    "recpre.model_dynamic.SwinBlock": "models.blocks:SwinBlock",
    "recpre.model_dynamic.SandwichBlock": "models.blocks:SandwichBlock",
    "recpre.model_dynamic.SandwichBlockSwin": "models.variants:SandwichBlockSwin",
    "recpre.model_dynamic.RevTransformerPreNormBlock": "models.variants:RevTransformerPreNormBlock",
    "recpre.model_dynamic.TransformerPostNormBlockDiff": "models.variants:TransformerPostNormBlockDiff",
    "recpre.model_dynamic.TransformerPostNormBlockDiffSimplified": "models.variants:TransformerPostNormBlockDiffSimplified",
    "recpre.model_dynamic.TransformerPostNormPosBlock": "models.variants:TransformerPostNormPosBlock",
    "recpre.model_dynamic.ParallelGatedMLPSelfAttention": "models.variants:ParallelGatedMLPSelfAttention",
    "recpre.model_dynamic.GatedBlock": "models.variants:GatedBlock",
    "recpre.model_dynamic.ModulatedTransformerPostNormBlock": "models.variants:ModulatedTransformerPostNormBlock",
    "recpre.model_dynamic.Brick": "models.blocks:Brick",
    "recpre.model_dynamic.BrickLP": "models.blocks:BrickLP",
    "recpre.model_dynamic.precompute_freqs_cis": "ops.reference:freqs_cis_buffer",
    "recpre.model_dynamic.apply_rotary_emb_complex_like": "ops.reference:rope_interleaved",
    "recpre.model_dynamic.RecurrentGPT.randomized_iteration_sampler": "models.sampler:sample_recurrence",
    "recpre.model_dynamic.sample_gamma": "models.sampler:sample_gamma",
    "recpre.model_dynamic.sample_negative_binomial": "models.sampler:sample_negative_binomial",
    # ---- recpre/norms.py, init.py, misc.py, ops.py ----------------------------------------------------------------------
    "recpre.norms.RMSNorm": "models.blocks:RMSNorm",
    "recpre.norms.RMSNorm_llama": "models.blocks:RMSNorm",
    "recpre.norms.FusedRMSNorm": "models.blocks:RMSNorm",
    "recpre.config_dynamic.Config.norm_class": "models.blocks:make_norm",
    "recpre.norms.fused_rms_norm_fn": "ops.functional:rmsnorm",
    "recpre.init.Init": "models.init:Init",
    "recpre.init.get_factor_table": "models.init:strategy_table",
    "recpre.init.wrapped_trunc_normal": "models.init:trunc_normal_",
    "recpre.init.wrapped_trunc_ortho": "models.init:trunc_orthogonal_",
    "recpre.misc.precompute_freqs_cis_complex": "ops.rope_variants:complex_table",
    "recpre.misc.apply_rotary_emb_complex": "ops.rope_variants:rope_complex",
    "recpre.misc.apply_rotary_emb": "ops.reference:rope_interleaved",
    "recpre.misc.apply_rotary_emb_v2": "ops.reference:rope_interleaved",
    "recpre.ops.reference_torch": "ops.reference:linear_cross_entropy",
    "recpre.ops.LinearXentImplementation": "ops.functional:linear_cross_entropy",
    "recpre.ops.linear_cross_entropy": "ops.functional:linear_cross_entropy",
    # ---- attention back ends ----------------------------------------------------------------------------------------------
    # (select_attention_implementation: the provider / center / debias options are attributes of CausalSelfAttention)
    "recpre.attention_backends.interface.select_attention_implementation": "models.blocks:CausalSelfAttention",
    "recpre.attention_backends.pytorch.attention_computation_sdpa": "ops.functional:causal_attention",
    "recpre.attention_backends.cuda_flash_attention.attention_computation_flash": "ops.functional:causal_attention",
    "recpre.attention_backends.testing.baseline_attn": "ops.reference:causal_attention",
    "recpre.attention_backends.testing.bench_flash_attention": "utils.kernel_bench:bench_attn",
    # ---- recpre/raven_modeling_minimal.py, legacy file -----------------------------------------------------------------------
    "recpre.raven_modeling_minimal.RavenPreTrainedModel": "models.hf:RavenPreTrainedModel",
    "recpre.raven_modeling_minimal.RavenForCausalLM": "models.hf:RavenForCausalLM",
    "recpre.raven_modeling_minimal.CausalLMOutputRecurrentLatents": "models.hf:CausalLMOutputRecurrentLatents",
    "recpre.raven_modeling_minimal.GenerateDecoderOnlyOutput": "models.generation:GenerateOutput",
    "recpre.raven_modeling_minimal.HuginnDynamicCache": "models.kv_cache:RecurrentKVCache",
    "recpre.raven_modeling_minimal.HuginnStaticCache": "models.kv_cache:StaticRecurrentCache",
    "recpre.raven_modeling_minimal.PerIterationExitEvaluator": "models.exit_criteria:PerIterationExitEvaluator",
    "recpre.raven_modeling_minimal.NoOpExitEvaluator": "models.exit_criteria:NoOpExitEvaluator",
    "recpre.raven_modeling_minimal.EntropyDiffExitEvaluator": "models.exit_criteria:EntropyDiffExitEvaluator",
    "recpre.raven_modeling_minimal.KLExitEvaluator": "models.exit_criteria:KLExitEvaluator",
    "recpre.raven_modeling_minimal.MinKLExitEvaluator": "models.exit_criteria:MinKLExitEvaluator",
    "recpre.raven_modeling_minimal.ArgmaxStabilityExitEvaluator": "models.exit_criteria:ArgmaxStabilityExitEvaluator",
    "recpre.raven_modeling_minimal.LatentDiffExitEvaluator": "models.exit_criteria:LatentDiffExitEvaluator",
    "recpre.raven_modeling_minimal.CosineExitEvaluator": "models.exit_criteria:CosineExitEvaluator",
    "recpre.raven_modeling_minimal.NumStepsGenerator": "models.exit_criteria:NumStepsGenerator",
    "recpre.raven_modeling_minimal.get_adaptive_exit_evaluator": "models.exit_criteria:get_adaptive_exit_evaluator",
    "recpre.legacy_modeling_file.RavenForCausalLM": "models.legacy:RavenForCausalLM",
    # ---- recpre/optim.py, soap.py ---------------------------------------------------------------------------------------------
    "recpre.optim.get_param_groups": "optim.groups:get_param_groups",
    "recpre.optim.get_optimizer": "optim.registry:get_optimizer",
    "recpre.optim.ELLISAdam": "optim.ellis:ELLISAdam",
    "recpre.optim.LionW": "optim.others:LionW",
    "recpre.optim.SophiaG": "optim.others:SophiaG",
    "recpre.optim.Lilith": "optim.research:Lilith",
    "recpre.optim.IVON": "optim.research:IVON",
    "recpre.optim.ZeroShampooWithAdamGraftingOptimizer": "optim.research:ZeroShampooWithAdamGraftingOptimizer",
    "recpre.optim.OrthogonalNesterov": "optim.others:OrthogonalNesterov",
    "recpre.optim.zeroth_power_via_newtonschulz5": "optim.others:zeroth_power_via_newtonschulz5",
    "recpre.soap.SOAP": "optim.soap:SOAP",
    "recpre.optim.SimpleZeroRedundancyOptimizer": "optim.zero:SimpleZeroRedundancyOptimizer",
    # ---- data -----------------------------------------------------------------------------------------------------------------
    "recpre.huggingface_dataset.ParquetStreamPure": "data.datasets:ParquetStream",
    "recpre.huggingface_dataset.ParquetStream": "data.datasets:BufferShuffledParquet",
    "recpre.huggingface_dataset.HuggingfaceDataset": "data.datasets:TextRows",
    "recpre.huggingface_dataset.HuggingfaceCombinedDataset": "data.datasets:WeightedMixture",
    "recpre.huggingface_dataset.RandomTokensDataset": "data.datasets:RandomTokens",
    "recpre.data_loading_utils.generic_collate_fn": "data.collate:generic_collate_fn",
    "recpre.data_loading_utils.pass_text": "data.collate:pass_text",
    "recpre.data_loading_utils.concat_input_target": "data.collate:concat_input_target",
    "recpre.data_loading_utils.condition_input_supervise_target": "data.collate:condition_input_supervise_target",
    "recpre.data_loading_utils.apply_chat_template_supervise_all": "data.collate:apply_chat_template_supervise_all",
    "recpre.data_loading_utils.apply_chat_template_supervise_assistant":
        "data.collate:apply_chat_template_supervise_assistant",
    "recpre.data_loading_utils.apply_formatting": "data.collate:apply_formatting",
    "recpre.data_loading_utils.shift_inputs_and_labels": "data.collate:shift_inputs_and_labels",
    "recpre.data_scheduler_utils.DataScheduler": "data.scheduler:DataScheduler",
    "recpre.data_scheduler_utils.DataSchedulerTracker": "data.scheduler:DataSchedulerTracker",
    "recpre.data_scheduler_utils.GetScheduler": "data.scheduler:GetScheduler",
    "recpre.data_scheduler_utils.ConstWeight": "data.scheduler:ConstWeight",
    "recpre.data_scheduler_utils.StepWeight": "data.scheduler:StepWeight",
    "recpre.data_scheduler_utils.LinearWeight": "data.scheduler:LinearWeight",
    "recpre.data_scheduler_utils.CosineAnnealingWeight": "data.scheduler:CosineAnnealingWeight",
    "recpre.data_scheduler_utils.PiecewiseWeight": "data.scheduler:PiecewiseWeight",
    "recpre.data_scheduler_utils.BaseWeight": "data.scheduler:BaseWeight",
    "recpre.tokenizer.Tokenizer": "data.tokenizer:Tokenizer",
    "recpre.utils.apply_tld": "data.goldfish:apply_tld",
    "recpre.utils.hashint": "data.goldfish:hashint",
    "train.StatefulDataLoader": "data.loader:StatefulLoader",
    # ---- recpre/monitor.py ----------------------------------------------------------------------------------------------------
    "recpre.monitor.enable_monitoring_on_step": "runtime.monitor:enable_monitoring",
    "recpre.monitor.disable_monitoring_and_retrieve_metrics": "runtime.monitor:harvest_metrics",
    "recpre.monitor.track_gradient_metrics": "runtime.monitor:optimizer_telemetry",
    "recpre.monitor._reverse_engineer_adam_effective_lr": "runtime.monitor:adam_effective_lr",
    "recpre.monitor._get_num_params": "runtime.monitor:num_params",
    "recpre.monitor._estimate_num_flop_per_token": "runtime.monitor:estimate_flops_per_token",
    "recpre.monitor._actually_measure_flops": "runtime.monitor:measure_flops",
    "recpre.monitor._get_peak_flops": "runtime.monitor:peak_flops",
    "recpre.monitor.get_MFU_metrics": "runtime.monitor:mfu_metrics",
    "recpre.monitor.standalone_measure_peak_flops": "runtime.monitor:measure_peak_flops",
    # ---- recpre/utils.py ------------------------------------------------------------------------------------------------------
    "recpre.utils.LightningFabric": "parallel.fabric:Fabric",
    "recpre.utils.SimpleFabric": "parallel.fabric:Fabric",
    "recpre.utils._allreduce_chunk_stream": "parallel.collectives:FusedCollectives",
    "recpre.utils.find_multiple": "utils.helpers:find_multiple",
    "recpre.utils.num_parameters": "utils.helpers:num_parameters",
    "recpre.utils.reset_parameters": "utils.helpers:reset_parameters",
    "recpre.utils.check_valid_checkpoint_dir": "utils.helpers:check_valid_checkpoint_dir",
    "recpre.utils.extend_checkpoint_dir": "utils.helpers:extend_checkpoint_dir",
    "recpre.utils.copy_config_files": "utils.helpers:copy_config_files",
    "recpre.utils.flatten_dict": "utils.helpers:flatten_dict",
    "recpre.utils.capture_hparams": "utils.helpers:capture_hparams",
    "recpre.utils.save_hyperparameters": "utils.helpers:save_hyperparameters",
    "recpre.utils.save_config": "utils.helpers:save_config",
    "recpre.utils.parse_devices": "utils.helpers:parse_devices",
    "recpre.utils.get_default_supported_precision": "utils.helpers:get_default_supported_precision",
    "recpre.utils.map_old_state_dict_weights": "utils.helpers:map_old_state_dict_weights",
    "recpre.utils.slice_logits_remap_labels": "utils.helpers:slice_logits_remap_labels",
    "recpre.utils.CycleIterator": "utils.helpers:CycleIterator",
    "recpre.utils.param_count_estimator": "utils.helpers:param_count_estimator",
    "recpre.utils.get_abacus_param_groups": "utils.helpers:get_abacus_param_groups",
    "recpre.utils.LinearCrossEntropyLoss": "utils.helpers:LinearCrossEntropyLoss",
    "recpre.utils.ChunkedCE": "utils.extras:chunked_cross_entropy",
    "recpre.utils.chunked_cross_entropy": "utils.extras:chunked_cross_entropy",
    "recpre.utils.incremental_save": "utils.extras:incremental_save",
    "recpre.utils.batch_exact_match": "utils.extras:batch_exact_match",
    "recpre.utils.estimate_flops": "utils.extras:estimate_flops",
    "recpre.utils.flops_per_param": "utils.extras:flops_per_param",
    "recpre.utils.simple_gptneox_tflops": "utils.extras:gptneox_tflops",
    "recpre.utils.simple_axonn_tflops": "utils.extras:gated_mlp_tflops",
    "recpre.utils.choose_logger": "runtime.monitor:make_loggers",
    # ---- evaluation, conversion, serving, launch ----------------------------------------------------------------------------------
    "evaluate_raven.quick_checkpoint_eval.RecurrentGPTWrapper": "evaluate.lm_eval_wrapper:RecurrentLM",
    "evaluate_raven.quick_checkpoint_eval.quick_eval_check": "evaluate.local_lm_eval:quick_eval_check",
    "evaluate_raven.quick_checkpoint_eval.prepare_results": "evaluate.local_lm_eval:prepare_results",
    "evaluate_raven.local_lm_eval.cli_evaluate": "evaluate.local_lm_eval:main",
    "evaluate_raven.checkpoint_to_hf_converter.hf_implementation_test_and_upload":
        "evaluate.convert_to_hf:hf_implementation_test_and_upload",
    "evaluate_raven.checkpoint_to_hf_converter.mini_generate": "evaluate.convert_to_hf:greedy",
    "evaluate_raven.quick_chat_rec_compare.quick_chat_interface": "evaluate.chat_compare:main",
    "evaluate_raven.record_steps_in_bench.evaluate_with_steps": "evaluate.record_steps:evaluate_with_steps",
    "evaluate_raven.record_steps_in_bench.save_step_histogram": "evaluate.record_steps:save_step_histogram",
    "evaluate_raven.record_steps_in_bench.parse_gen_kwargs": "evaluate.record_steps:parse_gen_kwargs",
    "evaluate_raven.saturation_eval_dist.saturation_eval": "evaluate.saturation_eval:saturation_eval",
    "evaluate_raven.misc_benchmark_variants.hf_eval_adaptive_compute.HuginnWrapper": "evaluate.adaptive_eval:AdaptiveComputeLM",
    "vllm.raven_vllm.RavenForvLLM": "engine.decode:DecodeEngine",
    "vllm.raven_vllm.register": "engine.server:create_app",
    # ---- offline data preparation ---------------------------------------------------------------------------------------------------
    "scripts.tokenizer_generation.create_tokenizer": "data.prepare.tokenizer_train:train_tokenizer",
    "scripts.tokenizer_generation.get_manually_added_tokens": "data.prepare.tokenizer_train:manual_tokens",
    "scripts.tokenizer_generation.get_special_tokens": "data.prepare.special_tokens:special_token_ids",
    "scripts.data_processing_pipeline.get_unifying_formatter": "data.prepare.unify_filter:unify_row",
    "scripts.data_processing_pipeline.format_ftfy": "data.prepare.unify_filter:fix_text",
    "scripts.data_processing_pipeline.process_files": "data.prepare.unify_filter:process_source",
    "scripts.scalable_data_download.download_datasets_raw": "data.prepare.download:download_sources",
    "scripts.scalable_data_download.software_heritage_aws_download": "data.prepare.download:attach_blob_contents",
    "scripts.parquet_to_parquet_tokenizer.parquet_to_parquet_tokenization": "data.prepare.tokenize_pack:prepare",
    "scripts.parquet_to_parquet_shuffler.process_shards": "data.prepare.shuffle_shards:shuffle_shards",
    "scripts.parquet_to_parquet_dedup": "data.prepare.dedup:dedup_parquet",
    "scripts.parquet_token_counter.parquet_to_parquet_token_counter": "data.prepare.count_tokens:count_folder",
    "scripts.process_token_counts.count_tokens": "data.prepare.count_tokens:category_report",
    "scripts.compare_tokenizers.compare_tokenizations": "data.prepare.compare_tokenizers:compare",
    "scripts.compare_tokenizers.validate_tokenizers": "data.prepare.compare_tokenizers:validate_roundtrip",
    "scripts.classify_loops.capture_forward_latents": "data.prepare.loop_probe:capture_latents",
    "scripts.classify_loops.train_loop_predictor": "data.prepare.loop_probe:train_probe",
    "scripts.classify_loops.train_binary_loop_classification_sweep": "data.prepare.loop_probe:binary_sweep",
}


def _load(target: str) -> Any:
    module, _, attr = target.partition(":")
    return getattr(importlib.import_module(f"{_PKG}.{module}"), attr)


def resolve(reference_path: str) -> Any:
    """The object of this package that stands for ``reference_path`` (a key of ``REFERENCE_NAMES``)."""
    try:
        return _load(REFERENCE_NAMES[reference_path])
    except KeyError:
        raise KeyError(f"{reference_path!r} has no counterpart listed; known modules: "
                       f"{sorted({k.rsplit('.', 1)[0] for k in REFERENCE_NAMES})}") from None


def where(reference_path: str) -> str:
    """``package.module:attribute`` of the counterpart, without importing it."""
    return f"{_PKG}.{REFERENCE_NAMES[reference_path]}"


def _bare_names() -> dict[str, str]:
    seen: dict[str, set] = {}
    for key, target in REFERENCE_NAMES.items():
        seen.setdefault(key.rsplit(".", 1)[1], set()).add(target)
    return {name: next(iter(t)) for name, t in seen.items() if len(t) == 1}


def __getattr__(name: str) -> Any:          # ``reference_names.ParquetStreamPure``
    target = _bare_names().get(name)
    if target is None:
        raise AttributeError(f"no unique reference symbol named {name!r}")
    return _load(target)
