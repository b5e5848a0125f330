"""ZeRO-1-like optimizer-state sharding over the ranks of one node (recpre/optim.py:131-263).

Shard rule (positional "magic numbers" of the reference): param group 0 (weights) is dealt round-robin to local ranks
1..L-1 (``weights[r-1::L-1]``), group 1 (embeddings) lives on local rank 0, all further groups (norms, biases) are
replicated.  After the local step every owner broadcasts its parameters inside the node group.  Gradients and
parameters stay replicated; the state dict is per local rank.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch.optim import Optimizer


class SimpleZeroRedundancyOptimizer(Optimizer):
    verbose = False
    single_rank_return = False       # True: ``state_dict`` gathers every local rank's state on the node's first rank

    def __init__(self, params, optimizer_class, **kwargs):
        params = list(params)
        self.arg_lr = kwargs.get("lr")
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            self.local_optim_group = optimizer_class(params, **kwargs)
            self.local_rank, self.local_devices, self.node_root, self.local_pg = 0, 1, 0, None
        else:
            rank, world = dist.get_rank(), dist.get_world_size()
            n_dev = torch.cuda.device_count() if torch.cuda.is_available() else world
            self.local_devices = min(int(os.getenv("SLURM_NTASKS_PER_NODE", os.getenv("LOCAL_WORLD_SIZE", n_dev))), world)
            self.local_rank = int(os.getenv("LOCAL_RANK", rank % self.local_devices))
            node = rank // self.local_devices
            ranks = [r for r in range(world) if r // self.local_devices == node]
            self.node_root = ranks[0]
            self.local_pg = None
            for nd in range((world + self.local_devices - 1) // self.local_devices):  # every rank creates every group
                grp = dist.new_group(ranks=[r for r in range(world) if r // self.local_devices == nd])
                if nd == node:
                    self.local_pg = grp
            if self.local_devices < 2:
                raise ValueError("optimizer sharding needs at least two ranks per node")
            local_groups = []
            if self.local_rank == 0:
                local_groups.append(params[1])
            else:
                shard = dict(params[0])
                shard["params"] = params[0]["params"][self.local_rank - 1:: self.local_devices - 1]
                local_groups.append(shard)
            local_groups.extend(params[2:])
            self.local_optim_group = optimizer_class(local_groups, **kwargs)
            dist.barrier()
        super().__init__(params, {})

    def _sync_lr(self):
        # the training loop writes lr into self.param_groups; forward it to the local optimizer by group role
        if self.local_devices == 1:
            for src, dst in zip(self.param_groups, self.local_optim_group.param_groups):
                dst["lr"] = src["lr"]
            return
        first = self.param_groups[1] if self.local_rank == 0 else self.param_groups[0]
        self.local_optim_group.param_groups[0]["lr"] = first["lr"]
        for src, dst in zip(self.param_groups[2:], self.local_optim_group.param_groups[1:]):
            dst["lr"] = src["lr"]

    @torch.no_grad()
    def step(self, closure=None):
        self._sync_lr()
        self.local_optim_group.step(closure)
        self.sync_parameters()

    @torch.no_grad()
    def sync_parameters(self):
        if self.local_pg is None:
            return
        for p in self.param_groups[1]["params"]:
            dist.broadcast(p.data, src=self.node_root, group=self.local_pg)
        weights = self.param_groups[0]["params"]
        for i in range(self.local_devices - 1):
            for p in weights[i:: self.local_devices - 1]:
                dist.broadcast(p.data, src=self.node_root + i + 1, group=self.local_pg)

    @staticmethod
    def _cpu_state_dict(state_dict: dict) -> dict:
        out = {}
        for k, v in state_dict.items():
            if k == "state":
                out[k] = {pid: {n: (t.cpu() if torch.is_tensor(t) else t) for n, t in st.items()} for pid, st in v.items()}
            else:
                out[k] = v
        return out

    def state_dict(self, cpu_before_gather: bool = True):
        """``[local state]`` on every rank; with ``single_rank_return`` the node's first rank gets the list of all local
        states and the others an empty one (recpre/optim.py:212-236)."""
        local = self.local_optim_group.state_dict()
        if self.local_pg is None:
            return [self._cpu_state_dict(local)]
        if not self.single_rank_return:
            return [local]
        local = self._cpu_state_dict(local) if cpu_before_gather else local
        states = [None] * self.local_devices if self.local_rank == 0 else None
        dist.gather_object(local, states, dst=self.node_root, group=self.local_pg)
        if self.local_rank == 0:
            return states if cpu_before_gather else [self._cpu_state_dict(s) for s in states]
        return [{"state": {}, "param_groups": []}]

    def load_state_dict(self, state_dict):
        if isinstance(state_dict, list):
            state_dict = state_dict[self.local_rank] if (self.single_rank_return and len(state_dict) > 1) \
                else state_dict[0]
        self.local_optim_group.load_state_dict(state_dict)

    def __repr__(self) -> str:
        return type(self).__name__ + repr(self.local_optim_group)
