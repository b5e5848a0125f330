"""Process-group fabric: one process per GPU, ``torch.distributed`` (NCCL on GPUs, gloo on CPU) for rendezvous
and control traffic, and pluggable gradient synchronisation.

Counterpart of the reference's ``SimpleFabric`` (recpre/utils.py:1072-1289): same responsibilities (device set-up,
seeding, gradient all-reduce after the last micro-batch of an accumulation window, scalar reductions, barrier,
broadcast, rank-0 printing, save/load helpers) with a different data path on GPUs:

* ``grad_sync="chunked"``  -- the reference's semantics: sum-all-reduce of fp32 chunks of at most 64 MiB followed
  by a division by the world size (recpre/utils.py:1004-1043).  Used on CPU/gloo and as the NCCL baseline.
* ``grad_sync="flat"``     -- one NCCL all-reduce per flat optimizer-group buffer (no pack/unpack copies); the
  1/world factor is folded into the fused optimizer kernel.
* ``grad_sync="p2p"``      -- hand-written kernels over NVLink peer memory on symmetric buffers: bucketed reduce-scatter
  overlapped with the backward pass, sharded optimizer state, update that stores the new bf16 weights into every rank
  (``parallel.p2p``).  One node, at most 8 ranks; anything else falls back to ``flat`` with a notice.
* ``grad_sync="ddp"``      -- torch ``DistributedDataParallel`` around the model (bucketed all-reduce inside backward,
  ``find_unused_parameters`` for the untracked recurrences): the reference's alternative path
  (recpre/utils.py:1154-1155); used with ``torch.optim`` optimizers (the engine's ``torch`` mode).
* ``grad_sync="p2p-host"`` -- the bookkeeping of ``p2p`` on ``torch.distributed`` collectives (any backend; tests).
* ``grad_sync="zero3"``    -- as ``p2p`` with fp32 masters sharded as well and the updated bf16 weights pulled by the
  next forward pass (all-gather fused into the first consuming GEMM for the row-sharded QKV / gate-up weights).
"""
from __future__ import annotations

import datetime
import os
from contextlib import contextmanager

import torch
import torch.distributed as dist

CHUNK_ELEMS = 64 * 1024 * 1024 // 4  # 64 MiB of fp32


class Fabric:
    def __init__(self, device: torch.device, rank: int = 0, world_size: int = 1, local_rank: int = 0,
                 grad_sync: str = "flat", precision: str = "bf16-mixed"):
        self.device, self.global_rank, self.world_size, self.local_rank = device, rank, world_size, local_rank
        self.grad_sync = grad_sync
        self.precision = precision
        self.flat_groups = []
        self._loggers: list = []
        self._p2p = None
        self._p2p_alloc = None
        self.no_sync = False

    # -- construction ----------------------------------------------------------------------
    @classmethod
    def single(cls, device) -> "Fabric":
        return cls(torch.device(device))

    @classmethod
    def from_env(cls, backend: str | None = None, grad_sync: str | None = None, timeout_s: int = 900,
                 precision: str = "bf16-mixed") -> "Fabric":
        """Read RANK / WORLD_SIZE / LOCAL_RANK (or their SLURM equivalents) and join the process group."""
        env = os.environ
        rank = int(env.get("RANK", env.get("SLURM_PROCID", 0)))
        world = int(env.get("WORLD_SIZE", env.get("SLURM_NTASKS", 1)))
        local = int(env.get("LOCAL_RANK", env.get("SLURM_LOCALID", 0)))
        use_cuda = torch.cuda.is_available() and backend != "gloo"
        device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(device)
        if world > 1 and not dist.is_initialized():
            env.setdefault("MASTER_ADDR", "127.0.0.1")
            env.setdefault("MASTER_PORT", "29500")
            backend = backend or ("nccl" if use_cuda else "gloo")
            kwargs = {"device_id": device} if backend == "nccl" else {}
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        sync = grad_sync or ("flat" if use_cuda else "chunked")
        if sync in ("p2p", "zero3") and world > 1:
            local_world = int(env.get("LOCAL_WORLD_SIZE", env.get("SLURM_NTASKS_PER_NODE", world)))
            if not use_cuda or local_world != world or world > 8:
                if rank == 0:
                    print(f"grad_sync={sync!r} needs all ranks on one node (<= 8 GPUs); world {world}, "
                          f"{local_world} per node: using the NCCL 'flat' path", flush=True)
                sync = "flat" if use_cuda else "chunked"
        return cls(device, rank, world, local, sync, precision)

    # -- basic collectives -----------------------------------------------------------------
    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1 and dist.is_initialized()

    def barrier(self) -> None:
        if self.is_distributed:
            if self.device.type == "cuda":
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    def all_reduce(self, t, reduce_op: str = "mean") -> torch.Tensor:
        if not torch.is_tensor(t):                    # plain numbers (and lists of them) are accepted, as there
            t = torch.as_tensor(t, dtype=torch.float32, device=self.device)
        if not self.is_distributed:
            return t
        t = t.clone()
        op = {"sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN,
              "max": dist.ReduceOp.MAX}[reduce_op]
        dist.all_reduce(t, op=op)
        if reduce_op == "mean":
            t = t / self.world_size
        return t

    def broadcast(self, obj, src: int = 0):
        if not self.is_distributed:
            return obj
        if torch.is_tensor(obj):
            dist.broadcast(obj, src)
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src)
        return box[0]

    def print(self, *a, ranks=(0,), **k) -> None:
        if self.global_rank in ranks:
            print(*a, **k, flush=True)

    def seed_everything(self, seed: int | None = None, workers: bool = False) -> int:
        import random

        import numpy as np

        if seed is None:
            seed = int(os.environ.get("PL_GLOBAL_SEED", 0))
        seed = int(seed) % (2 ** 32)
        os.environ["PL_GLOBAL_SEED"] = str(seed)
        os.environ["PL_SEED_WORKERS"] = str(int(workers))
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)
        return seed

    @contextmanager
    def no_backward_sync(self, model=None, enabled: bool = True):
        """``with fabric.no_backward_sync(model, enabled=accumulating):`` -- gradients of the micro-batches inside stay
        local (``no_backward_sync(flag)`` without a model is accepted too)."""
        if isinstance(model, bool):
            model, enabled = None, model
        prev, self.no_sync = self.no_sync, bool(enabled)
        try:
            yield
        finally:
            self.no_sync = prev

    # -- the hand-written-loop interface of the reference's fabric (recpre/utils.py:1072-1289) --------------------------
    # For loops that own their model and a torch.optim optimizer:  model = fabric.setup(model); ...;
    # fabric.backward(loss, model=model); fabric.clip_gradients(model, opt, max_norm=1.0); opt.step().  The fused engine
    # (runtime.engine.TrainEngine) does not go through these.
    verbose = False

    def launch(self) -> None:
        pass

    @property
    def rank(self) -> int:
        return self.global_rank

    @property
    def local_device(self) -> torch.device:
        return self.device

    @property
    def strategy(self) -> str:
        return self.strategy_name

    @property
    def strategy_name(self) -> str:
        return {"p2p": "B200P2P", "zero3": "B200Sharded", "ddp": "DDP"}.get(self.grad_sync, "SimpleDDP")

    @property
    def local_devices(self) -> int:
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("SLURM_NTASKS_PER_NODE", self.world_size)))
        return max(min(per_node, self.world_size), 1)

    @property
    def logger(self):
        return self._loggers[0]

    def log_dict(self, metrics: dict, step: int | None = None) -> None:
        """Rank 0 hands the metrics (tensors turned into numbers) to every logger's ``log_metrics``."""
        if self.global_rank != 0:
            return
        plain = {k: (v.item() if torch.is_tensor(v) and v.numel() == 1 else v) for k, v in metrics.items()}
        for logger in self._loggers:
            logger.log_metrics(metrics=plain, step=step)

    def log_to_summary(self, dict_of_values: dict) -> None:
        if self.global_rank == 0 and self._loggers:
            summary = getattr(getattr(self.logger, "experiment", None), "summary", None)
            if summary is not None:
                for key, value in dict_of_values.items():
                    summary[key] = value
            elif hasattr(self.logger, "log_metrics"):
                self.logger.log_metrics(metrics={f"summary/{k}": v for k, v in dict_of_values.items()}, step=None)

    def log_chart(self, dict_of_charts: dict) -> None:
        if self.global_rank == 0 and self._loggers and hasattr(getattr(self.logger, "experiment", None), "log"):
            self.logger.experiment.log(dict_of_charts)

    def setup_dataloaders(self, train_dataloader, val_dataloader=None):
        return train_dataloader, val_dataloader

    def setup(self, model, compile: bool = False):
        """Move the model to this rank's device (and remember it for ``no_backward_sync`` / ``backward``).  ``compile``
        is accepted and ignored: the kernels behind the model's ops are compiled ahead of time."""
        self.model_ref = model.to(self.device)
        return self.model_ref

    def setup_optimizers(self, optimizers):
        return optimizers

    def backward(self, loss, model=None) -> None:
        """``loss.backward()`` and, outside ``no_backward_sync``, the averaging of the gradients over the ranks."""
        loss.backward()
        model = model if model is not None else getattr(self, "model_ref", None)
        if not self.no_sync and self.is_distributed and model is not None:
            self.all_reduce_gradients([p for p in model.parameters()])

    def clip_gradients(self, model, optimizer=None, max_norm: float = 1.0, error_if_nonfinite: bool = False):
        return torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm, norm_type=2.0,
                                              error_if_nonfinite=error_if_nonfinite)

    def get_prefix_for_checkpoint(self) -> str:
        from ..runtime.checkpoint import PREFIX

        return PREFIX

    def save(self, checkpoint_file_location: str, state: dict, overwrite: bool = True, strict: bool = False) -> None:
        """``{location}_{local_rank}.pth`` written by the ranks of the first node; ``model``, ``optimizer`` and the
        train loader entries are stored as their ``state_dict()`` (formed on every rank: they may be collective)."""
        payload = {}
        for key, value in state.items():
            payload[key] = value.state_dict() if (key in ("optimizer", "model") or "train_dataloader" in key) else value
        if self.global_rank >= self.local_devices:
            return
        folder = os.path.dirname(checkpoint_file_location)
        if folder:
            os.makedirs(folder, exist_ok=True)
        path = f"{checkpoint_file_location}_{self.local_rank}.pth"
        if os.path.exists(path) and not overwrite:
            raise ValueError(f"Checkpoint {path} already exists")
        tmp = path + ".tmp"
        torch.save(payload, tmp)
        os.replace(tmp, path)
        if self.verbose:
            print(f"Rank {self.global_rank} - local {self.local_rank} saved {path}.", flush=True)

    def load(self, checkpoint_file_location: str, state: dict, strict: bool = False) -> None:
        path = f"{checkpoint_file_location}_{self.local_rank}.pth"
        checkpoint = torch.load(path, map_location="cpu", weights_only=False)
        for key, value in checkpoint.items():
            if key in ("optimizer", "model") or "train_dataloader" in key:
                state[key].load_state_dict(value)
            elif key not in ("tokenizer", "val_dataloader"):
                state[key] = value

    @contextmanager
    def init_module(self, empty_init: bool = False):
        yield None

    # -- gradient synchronisation ----------------------------------------------------------
    @property
    def uses_p2p(self) -> bool:
        return self.grad_sync in ("p2p", "zero3") and self.is_distributed and self.device.type == "cuda"

    @property
    def shards_masters(self) -> bool:
        return self.grad_sync == "zero3" and self.uses_p2p

    @property
    def pulls_parameters(self) -> bool:
        """Updated bf16 weights are pulled by the next forward pass (bucket by bucket on a side stream, QKV / gate-up
        inside their first GEMM) instead of being pushed to every rank by the update kernel.  Always so when the fp32
        masters are sharded; for the replicated mode it is a switch (``B200_PULL_PARAMS=1``)."""
        return self.shards_masters or (self.uses_p2p and os.environ.get("B200_PULL_PARAMS", "0") == "1")

    def buffer_allocator(self, group_index: int):
        """Allocator for the flat buffers of optimizer group ``group_index`` (symmetric memory in p2p mode)."""
        if not self.uses_p2p:
            return None
        if self._p2p_alloc is None:
            from .p2p import P2PAllocator

            self._p2p_alloc = P2PAllocator(self)
        return lambda kind, numel, dtype: self._p2p_alloc(group_index, kind, numel, dtype)

    def register_flat_groups(self, groups, model=None, optimizer=None) -> None:
        self.flat_groups = groups
        if self.grad_sync == "p2p-host" and self.is_distributed:
            # the sharded step with torch.distributed collectives instead of the NVLink kernels (CPU / gloo): the
            # same ownership, buckets and optimizer-state layout, used to check the host-side logic
            from .p2p import ShardedStepper

            self._p2p = ShardedStepper(self, groups, optimizer, model, backend="torch")
        if self.uses_p2p:
            from .p2p import AgHandle, ShardedStepper

            self._p2p = ShardedStepper(self, groups, optimizer, model, zero3=self.pulls_parameters,
                                       allocator=self._p2p_alloc)
            if self.pulls_parameters:
                # the big row-sharded projections are gathered by their first GEMM of a step
                for gi, g in enumerate(groups[:1]):
                    for t, (name, p) in enumerate(zip(g.names, g.params)):
                        if name.endswith(("attn.Wqkv.weight", "mlp.fc.weight")) and p.dim() == 2:
                            h = AgHandle(self._p2p, gi, t)
                            if h.usable:
                                p._ag = h

    def fused_reduce_and_step(self, optimizer, max_norm: float, grad_scale: float, do_update: bool) -> bool:
        """Run the fused reduce-scatter + sharded update + parameter push when available."""
        if self._p2p is None:
            return False
        self._p2p.step(optimizer, max_norm, grad_scale, do_update)
        return True

    def begin_backward(self, model, accumulating: bool) -> None:
        """Called before the forward pass of every micro-batch: arms the overlap scheduler (bucket reductions fired
        from the model's phase hooks during backward) and starts the parameter gathers of the sharded mode."""
        if self._p2p is not None:
            self._p2p.begin_step(model, accumulating)

    def reduce_gradients(self, optimizer) -> bool:
        """Sum the flat gradient buffers over ranks.  Returns True when the squared norm of the reduced
        gradients has already been written to ``optimizer.gnorm_sq`` by a fused path."""
        if not self.is_distributed:
            return False
        for g in self.flat_groups:
            if self.grad_sync == "chunked":
                for s in range(0, g.grad.numel(), CHUNK_ELEMS):
                    dist.all_reduce(g.grad[s:s + CHUNK_ELEMS])
            else:
                dist.all_reduce(g.grad)
        return False

    def all_reduce_gradients(self, params) -> None:
        """Reference semantics for unflattened parameters: pack gradients into fp32 chunks of at most 64 MiB,
        sum-all-reduce each chunk, divide by the world size, scatter back (recpre/utils.py:1004-1043)."""
        if not self.is_distributed or self.no_sync:
            return
        grads = [p.grad for p in params if p.grad is not None]
        if not grads:
            return
        batch, size = [], 0
        for g in grads:
            n = g.numel()
            if batch and size + n > CHUNK_ELEMS:
                self._reduce_batch(batch)
                batch, size = [], 0
            if n > CHUNK_ELEMS:
                flat = g.view(-1)
                for s in range(0, n, CHUNK_ELEMS):
                    piece = flat[s:s + CHUNK_ELEMS]
                    buf = piece.float()
                    dist.all_reduce(buf)
                    piece.copy_(buf / self.world_size)
                continue
            batch.append(g)
            size += n
        if batch:
            self._reduce_batch(batch)

    def _reduce_batch(self, batch) -> None:
        flat = torch.cat([g.reshape(-1).float() for g in batch])
        dist.all_reduce(flat)
        flat /= self.world_size
        off = 0
        for g in batch:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n

    def sync_parameters(self) -> None:
        """Parameter-sharded mode: complete the local bf16 weights outside a training step (validation, export)."""
        if self._p2p is not None:
            self._p2p.sync_parameters()

    def device_status(self) -> int:
        """Status word of the kernels' bounded waits on this rank (0: no wait ran out).  Synchronises the device, so the
        training loop reads it only where it synchronises anyway."""
        if self.device.type != "cuda":
            return 0
        from ..ops import cuda as K

        return K.check_device_status()

    # -- teardown --------------------------------------------------------------------------
    def shutdown(self) -> None:
        if self._p2p is not None:
            self._p2p.close()
            self._p2p = None
        if dist.is_initialized():
            dist.destroy_process_group()
