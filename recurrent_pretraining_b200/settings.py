"""Run settings: one dataclass whose field names are the YAML keys / ``--flags`` of the training CLI.

The field set, defaults and derived quantities follow the reference's ``CLISettings`` (recpre/settings.py:81-297) so
that its launch YAMLs load unchanged.  The loader is self-contained (the reference relies on jsonargparse):
``--config=file.yaml`` loads a file, any ``--field=value`` / ``--nested.field=value`` overrides it, values are parsed
as YAML scalars.  Fields added by this framework are grouped at the end and default to "off".
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional

import yaml


@dataclass
class HuggingfaceConfig:
    """A stock Hugging Face architecture as the training model (``model_impl: huggingface`` in the reference,
    recpre/settings.py:14-43): built from its config (``checkpoint`` folder or hub ``name``), random weights.  It trains
    through the engine's ``torch`` mode (library kernels); the native kernels serve the recurrent model family."""
    name: str
    checkpoint: Optional[str] = None
    block_size: Optional[int] = None
    strategy: Optional[str] = None
    abacus_ids: list = field(default_factory=lambda: list(range(10)))

    def construct_model(self, objective=None, gradient_checkpointing: bool = False, **kwargs):
        from transformers import AutoConfig, AutoModelForCausalLM

        model = AutoModelForCausalLM.from_config(AutoConfig.from_pretrained(self.checkpoint or self.name))
        if gradient_checkpointing:
            model.gradient_checkpointing_enable()
        return model


@dataclass
class DataEntry:
    type: str = "rngds"  # hfds | pqds | pqds-pure | rngds
    prefix: str = ""
    weight: int = 1
    data_signature: Optional[dict] = None
    name: Optional[str] = None
    data_dir: Optional[str] = None
    text_key: Optional[str] = None
    repetitions: Optional[int] = None
    max_epoch: Optional[int] = None
    scheduler: Optional[tuple] = None
    return_data_id: bool = False


@dataclass
class GoldfishConfig:
    k_token_loss_dropout: int = 4
    start_position: int = 0
    context_width: int = 13
    strategy: Optional[str] = None  # None | static | seeded_random | hash-table | hash-avalanche


@dataclass
class FabricConfig:
    optimize_communication: bool = False
    all_reduce_dtype: Optional[str] = None
    row_tensor_parallel_size: int = 1
    col_tensor_parallel_size: int = 1
    depth_tensor_parallel_size: int = 1
    optim_sharding: bool = False
    allow_optim_fusion: bool = False
    use_apex_adamw: bool = False
    fsdp_use_original_params: bool = False


def _default_optim():
    return {"lr": 4e-4, "weight_decay": 0.1, "betas": (0.9, 0.95), "eps": 1e-8}


@dataclass
class CLISettings:
    # main
    run_name: str = "default-run"
    out_dir: Optional[str] = None
    resume: bool = True
    max_tokens: int = 1_000_000_000_000
    max_steps: Optional[int] = None
    seed: int = 1337
    # model
    model_name: str = "tiny-llama-1.1b"
    model_impl: str = "recpre"
    block_size: int = 2048
    ignore_block_size_mismatch: bool = False
    model_checkpoint: Optional[str] = None
    doc_block_attn: bool = False
    cache_attn: bool = False
    eod_token: Optional[str] = None
    # optimisation
    world_batch_size: int = 2048
    batch_size_ramp: int = 0
    optimizer: str = "AdamW"
    optim_config: dict = field(default_factory=_default_optim)
    grad_clip: float = 1.0
    warmup_steps: int = 0
    cooldown_steps: int = 0
    lr_schedule: str = "cosine"
    min_lr: float = 4e-5
    no_weight_decay_for_bias_and_norm_params: bool = False
    # objective
    label_smoothing: float = 0.0
    z_regularization: float = 0.0
    goldfish: GoldfishConfig = field(default_factory=GoldfishConfig)
    # backend
    fabric_strategy: str = "ddp"  # simple-ddp | ddp | single | fsdp-* | axonn_tp | zero (sharded mode of this framework)
    fabric_precision: str = "bf16-mixed"
    fabric_use_lightning_environment: bool = False
    fabric: FabricConfig = field(default_factory=FabricConfig)
    micro_batch_size: int = 4
    compile_model: bool = False
    matmul_precision: str = "high"
    dataloader_num_workers: int = 0
    n_chunks: int = 4
    gradient_checkpointing: bool = False
    allow_nonfinite_loss: bool = False
    compiled_autograd: bool = False
    compile_optimizer: bool = False
    dynamo_ddp_config: str = "ddp_optimizer"
    loss_guardrail_active: bool = False
    skip_nonfinite_grads: bool = False
    fail_instead_of_recompile: bool = False
    # logging
    logger_name: str = "wandb"
    logger_project: str = "tinyllama"
    data_telemetry: bool = False
    model_telemetry: bool = True
    shape_watching_steps: int = 3
    log_step_interval: int = 1
    eval_iters: int = 100
    save_step_interval: int = 2000
    eval_step_interval: int = 2000
    save_first_step: bool = False
    save_last_step: bool = False
    save_n_min_before_job_done: Optional[int] = None
    measure_utilization: bool = True
    partial_depth_eval: list = field(default_factory=list)
    # data
    shuffle_filenames: bool = True
    shuffle_blocks: bool = True
    pad_to_block_size: bool = False
    add_bos: bool = True
    add_eos: bool = True
    data_signature: dict = field(default_factory=lambda: {"keys": ["text"], "format_fn": "pass_text"})
    collate_checks_enabled: bool = True
    all_block_size_tensors: bool = False
    use_chat_template: bool = False
    data_config: Any = field(default_factory=lambda: {"train_data": [DataEntry("rngds", "random")],
                                                      "val_data": [DataEntry("rngds", "random")]})
    train_data_dir: str = ""
    val_data_dir: str = ""
    tokenizer_path: str = ""
    model_overwrite: dict = field(default_factory=dict)
    # ---- added by this framework ----
    grad_sync: Optional[str] = None        # chunked | flat | p2p (default: p2p on >1 GPU, chunked on CPU)
    skip_first_optimizer_step: bool = True  # the reference never applies the first optimizer step of a run
    state_init_scale: float = 1.0

    # ------------------------------------------------------------------------------------------
    def __post_init__(self):
        if isinstance(self.goldfish, dict):
            self.goldfish = GoldfishConfig(**self.goldfish)
        if isinstance(self.fabric, dict):
            self.fabric = FabricConfig(**self.fabric)
        if self.out_dir is None:
            self.out_dir = os.getenv("OUTPUT_DIR", "NOT_FOUND")
        if self.out_dir == "NOT_FOUND":
            raise ValueError("out_dir must be given (or $OUTPUT_DIR set)")
        self.data_config = self._validate_data_config()
        self.train_data_dir = os.path.expandvars(self.train_data_dir or "")
        self.val_data_dir = os.path.expandvars(self.val_data_dir or "")
        for e in self.data_config["train_data"] + self.data_config.get("val_data", []):
            if e.data_dir is not None:
                e.data_dir = os.path.expandvars(e.data_dir)
        tp = self.fabric
        if max(tp.depth_tensor_parallel_size, tp.row_tensor_parallel_size, tp.col_tensor_parallel_size) > 1:
            raise ValueError("tensor parallelism is delegated to AxoNN in the reference and is not provided here")
        self._parse_environment_variables()
        self.node_batch_size = self.world_batch_size // self.num_nodes
        self.loader_block_size = self.block_size + 1
        self.batch_size = self.node_batch_size // self.devices
        if self.batch_size_ramp == 0:
            self.gradient_accumulation_steps = self.batch_size // self.micro_batch_size
        else:
            self.gradient_accumulation_steps = 1
        self.replicas = self.devices * self.num_nodes
        self.dataset_names = [e.prefix for e in self.data_config["train_data"]]
        self.train_dataset_prefixes = list(self.dataset_names)
        self.val_dataset_prefixes = [e.prefix for e in self.data_config.get("val_data", [])]
        # filled in by the trainer at start-up (recpre/settings.py:226-228)
        self.global_total_time, self.max_tokens_per_device, self.tokens_per_step = 0, 0, 0
        self._validate_args()
        from .config import ModelConfig

        overrides = dict(self.model_overwrite)
        if self.state_init_scale != 1.0:
            overrides.setdefault("state_init_scale", self.state_init_scale)
        self.model_config = ModelConfig.from_name(self.model_name, **overrides)
        self.model_config.strategy = self.fabric_strategy
        if self.max_steps is None:
            # micro-steps per device, as the reference derives them at start-up (train.py:268-271)
            self.max_tokens_per_device = self.max_tokens // max(self.replicas, 1)
            self.tokens_per_step = self.micro_batch_size * self.block_size
            self.max_steps = max(int(self.max_tokens_per_device // self.tokens_per_step), 1)

    def _validate_args(self):
        if not ((self.max_steps is not None) ^ (self.max_tokens > 0)):
            raise ValueError(f"only max_steps ({self.max_steps}) xor max_tokens ({self.max_tokens}) can be specified")
        if len(set(self.dataset_names)) != len(self.data_config["train_data"]):
            raise ValueError("please provide different names for each subset")
        if self.gradient_accumulation_steps <= 0:
            raise ValueError("derived gradient_accumulation_steps must be > 0")
        per_step = self.micro_batch_size * self.devices * self.num_nodes
        if self.batch_size_ramp == 0:
            if self.world_batch_size != per_step * self.gradient_accumulation_steps:
                raise ValueError("world batch size should be: micro_batch_size * gradient_accumulation_steps * "
                                 "devices * num_nodes")
        elif self.world_batch_size % per_step:
            raise ValueError("world_batch_size must be a multiple of micro_batch_size * devices * num_nodes")

    def _parse_environment_variables(self):
        env = os.getenv
        self.SLURM_JOB_ID = int(env("SLURM_JOB_ID", 0))
        self.SLURM_ARRAY_JOB_ID = int(env("SLURM_ARRAY_JOB_ID", 0))
        self.SLURM_ARRAY_TASK_ID = int(env("SLURM_ARRAY_TASK_ID", 0))
        self.SLURM_ARRAY_TASK_COUNT = int(env("SLURM_ARRAY_TASK_COUNT", 1))
        self.MASTER_ADDR = env("MASTER_ADDR", "127.0.0.1")
        self.MASTER_PORT = int(env("MASTER_PORT", 0))
        self.WORLD_SIZE = int(env("SLURM_NTASKS", env("WORLD_SIZE", 1)))
        self.RANK = int(env("SLURM_PROCID", env("RANK", 0)))
        self.num_nodes = int(env("SLURM_JOB_NUM_NODES", 1))
        per_node = env("SLURM_NTASKS_PER_NODE", env("LOCAL_WORLD_SIZE"))
        if per_node is not None:
            self.devices = int(per_node)
        else:
            self.devices = max(self.WORLD_SIZE // self.num_nodes, 1)

    def _validate_data_config(self) -> dict:
        cfg = self.data_config
        if isinstance(cfg, str):
            with open(cfg) as f:
                cfg = json.load(f)
        out = {}
        for key in ("train_data", "val_data"):
            out[key] = [e if isinstance(e, DataEntry) else DataEntry(**e) for e in cfg.get(key, [])]
        return out

    # ------------------------------------------------------------------------------------------
    def to_dict(self) -> dict:
        d = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if dataclasses.is_dataclass(v):
                v = dataclasses.asdict(v)
            elif f.name == "data_config":
                v = {k: [dataclasses.asdict(e) for e in lst] for k, lst in v.items()}
            d[f.name] = v
        return d

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2, default=str)


_SCI = __import__("re").compile(r"^[+-]?(\d+\.?\d*|\.\d+)[eE][+-]?\d+$")


def _coerce(v):
    """YAML 1.1 reads ``4e-5`` as a string; turn such scalars (and ``1_000`` style ints) into numbers."""
    if isinstance(v, str):
        if _SCI.match(v):
            return float(v)
        return v
    if isinstance(v, dict):
        return {k: _coerce(x) for k, x in v.items()}
    if isinstance(v, list):
        return [_coerce(x) for x in v]
    return v


def _set_dotted(d: dict, key: str, value) -> None:
    parts = key.split(".")
    for p in parts[:-1]:
        d = d.setdefault(p, {})
    d[parts[-1]] = value


def parse_cli(argv: list[str]) -> CLISettings:
    """``--config=x.yaml`` (repeatable; later files win) followed by ``--key=value`` / ``--a.b=value`` overrides."""
    merged: dict = {}
    overrides = []
    it = iter(argv)
    for tok in it:
        if not tok.startswith("--"):
            raise SystemExit(f"unexpected argument {tok!r}")
        if "=" in tok:
            key, val = tok[2:].split("=", 1)
        else:
            key, val = tok[2:], next(it, "true")
        if key == "config":
            with open(val) as f:
                loaded = _coerce(yaml.safe_load(f) or {})
            merged.update(loaded)
        else:
            overrides.append((key, _coerce(yaml.safe_load(val))))
    for key, val in overrides:
        _set_dotted(merged, key, val)
    known = {f.name for f in dataclasses.fields(CLISettings)}
    unknown = set(merged) - known
    if unknown:
        raise SystemExit(f"unknown settings: {sorted(unknown)}")
    if "optim_config" in merged and "betas" in merged["optim_config"]:
        merged["optim_config"]["betas"] = tuple(merged["optim_config"]["betas"])
    return CLISettings(**merged)
