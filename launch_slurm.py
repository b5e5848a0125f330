#!/usr/bin/env python
"""SLURM launch-file generator for multi-node runs on NVIDIA clusters (one task per node, torchrun inside, one
process per GPU, NCCL over NVLink inside a node and over the cluster fabric between nodes).

Functional counterpart of the reference's Frontier launcher (launch_frontier.py:213-320 sbatch assembly, :359-580
job arrays / chains, :582-619 interactive allocation, :622-733 CLI).  The AMD/Slingshot specifics (module loads, RCCL
plugin paths, sbcast of a conda archive) are replaced by what a B200 cluster needs: NCCL environment, the in-tree
kernel library build on the first node, and a per-node torchrun.

    python launch_slurm.py --config launch_configs/nebel_dp_8xb200.yaml --nodes 4 --budget_hours 12 --dryrun
"""
from __future__ import annotations

import argparse
import getpass
import os
import secrets
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field

HERE = os.path.dirname(os.path.abspath(__file__))


def nccl_environment(disable_net_gdr: bool = False, debug: bool = False) -> dict:
    """Environment of every rank.  NVLS (in-switch reduction) stays on for the NCCL paths; the framework's own fused
    kernels use plain peer loads/stores and do not depend on it."""
    env = {
        "OMP_NUM_THREADS": "8",
        "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",
        "NCCL_DEBUG": "INFO" if debug else "WARN",
        "NCCL_IB_TIMEOUT": "22",
        "NCCL_SOCKET_IFNAME": "^lo,docker",
        "CUDA_DEVICE_MAX_CONNECTIONS": "8",
        "PYTHONFAULTHANDLER": "1",
        "TOKENIZERS_PARALLELISM": "false",
    }
    if disable_net_gdr:
        env["NCCL_NET_GDR_LEVEL"] = "0"
    return env


def snapshot_working_tree(dest_dir: str | None = None, name: str = "repo_snapshot") -> str:
    """Freeze the code a queued job will run: tar the tracked and untracked-but-not-ignored files of this repository
    (``git ls-files``) into ``<dest_dir>/<name>.tar.gz`` under a top-level folder ``<name>/`` (the reference's
    ``compress_working_dir``, launch_frontier.py:88-101).  Later edits do not reach the job."""
    import subprocess
    import tarfile

    dest_dir = dest_dir or os.environ.get("WRKSPC", os.path.expanduser("~"))
    os.makedirs(dest_dir, exist_ok=True)
    out = os.path.join(dest_dir, f"{name}.tar.gz")
    listing = subprocess.run(["git", "ls-files", "--cached", "--others", "--exclude-standard"], cwd=HERE,
                             capture_output=True, text=True, check=True).stdout.splitlines()
    with tarfile.open(out, "w:gz") as tar:
        for rel in listing:
            full = os.path.join(HERE, rel)
            if os.path.isfile(full):
                tar.add(full, arcname=os.path.join(name, rel))
    return out


def stage_archives_script(archives, local_dir: str = "/tmp/${USER}/${SLURM_JOB_ID}", interval: int = 5) -> str:
    """Shell lines for the batch script that copy ``.tar.gz`` archives (code snapshot, packed environment) to
    node-local storage on every node with ``sbcast``, unpack them once per node and hold the other tasks of the node at
    a file barrier until that is done (launch_frontier.py:104-156)."""
    archives = [a for a in (archives or []) if a]
    if not archives:
        return ""
    for a in archives:
        if not a.endswith(".tar.gz"):
            raise ValueError(f"archive {a!r} is not a .tar.gz file")
    lines = [f'STAGE_DIR="{local_dir}"', 'srun --ntasks-per-node=1 mkdir -p "$STAGE_DIR"',
             f'echo "$(date -u) copying {",".join(os.path.basename(a) for a in archives)} to every node"']
    for a in archives:
        lines.append(f'sbcast -pf {shlex.quote(a)} "$STAGE_DIR/{os.path.basename(a)}" || {{ echo "sbcast failed"; exit 1; }}')
    unpack = " && ".join(f'tar -xzf "$STAGE_DIR/{os.path.basename(a)}" -C "$STAGE_DIR"' for a in archives)
    lines.append(f"srun --ntasks-per-node=1 bash -c '{unpack} && touch \"$STAGE_DIR/.unpacked\"'")
    lines.append(f'while [ ! -f "$STAGE_DIR/.unpacked" ]; do sleep {interval}; done')
    return "\n".join(lines) + "\n"


@dataclass
class SlurmJob:
    run_name: str
    python_script: str = "train.py"
    config: str | None = None
    extra_args: str = ""
    nodes: int = 1
    gpus_per_node: int = 8
    minutes: int = 120
    partition: str | None = None
    account: str | None = None
    qos: str | None = None
    email: str | None = None
    output_dir: str = field(default_factory=lambda: os.path.join(HERE, "outputs"))
    env: dict = field(default_factory=dict)
    custom_invocation: str | None = None
    dependency: str | None = None
    rebuild_kernels: bool = True
    archives: list = field(default_factory=list)     # .tar.gz files staged to node-local storage before the run
    run_from_snapshot: str | None = None             # top-level folder of the staged code snapshot to cd into
    environment: str | None = None                   # python environment: a directory, or a packed .tar.gz to stage
    sub_dir: str | None = None                       # folder under output_dir for logs and sbatch files (run name)
    proxy: str | None = None                         # http(s) proxy exported to the job (compute nodes without a route out)

    @property
    def log_dir(self) -> str:
        return os.path.join(self.output_dir, self.sub_dir or self.run_name, "slurm")

    def time_string(self) -> str:
        d, rem = divmod(self.minutes, 24 * 60)
        h, m = divmod(rem, 60)
        return f"{d}-{h:02d}:{m:02d}:00"

    def invocation(self) -> str:
        if self.custom_invocation:
            return self.custom_invocation
        cmd = [self.python_script]
        if self.config:
            cmd.append(f"--config={self.config}")
        cmd.append(f"--run_name={self.run_name}")
        cmd.append(f"--out_dir={self.output_dir}")
        return " ".join(shlex.quote(c) for c in cmd) + (" " + self.extra_args if self.extra_args else "")

    def sbatch_text(self, array: str | None = None) -> str:
        head = ["#!/bin/bash", f"#SBATCH --job-name={self.run_name}", f"#SBATCH --nodes={self.nodes}",
                "#SBATCH --ntasks-per-node=1", f"#SBATCH --gpus-per-node={self.gpus_per_node}",
                f"#SBATCH --time={self.time_string()}", "#SBATCH --exclusive",
                f"#SBATCH --output={self.log_dir}/%x_%A_%a.log" if array else f"#SBATCH --output={self.log_dir}/%x_%j.log",
                "#SBATCH --signal=B:USR1@180"]
        for key, val in (("partition", self.partition), ("account", self.account), ("qos", self.qos)):
            if val:
                head.append(f"#SBATCH --{key}={val}")
        if self.email:
            head += [f"#SBATCH --mail-user={self.email}", "#SBATCH --mail-type=FAIL,ARRAY_TASKS"]
        if array:
            head.append(f"#SBATCH --array={array}")
        if self.dependency:
            head.append(f"#SBATCH --dependency={self.dependency}")
        exports = "\n".join(f"export {k}={shlex.quote(str(v))}" for k, v in self.env.items())
        build = (f"srun --nodes=1 --ntasks=1 python -c 'import __graft_entry__ as g; g.build()'\n"
                 if self.rebuild_kernels else "")
        archives, activate = list(self.archives), ""
        if self.environment:
            env_path = self.environment
            if env_path.endswith(".tar.gz"):                 # packed environment: unpack on every node, use it there
                archives.append(env_path)
                env_path = '"$STAGE_DIR"/' + os.path.basename(env_path)[: -len(".tar.gz")]
            activate = (f'source {env_path}/bin/activate\n'
                        f'echo "$(date -u) activated {os.path.basename(self.environment)}"\n')
        if self.proxy:
            activate += "".join(f"export {v}={shlex.quote(self.proxy)}\n"
                                for v in ("http_proxy", "https_proxy", "HTTP_PROXY", "HTTPS_PROXY", "all_proxy"))
        stage = stage_archives_script(archives)
        workdir = f'"$STAGE_DIR/{self.run_from_snapshot}"' if (stage and self.run_from_snapshot) else shlex.quote(HERE)
        body = f"""
set -euo pipefail
{stage}cd {workdir}
{activate}{exports}
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))
echo "nodes: $SLURM_JOB_NODELIST  master: $MASTER_ADDR:$MASTER_PORT  started $(date)"
{build}srun --kill-on-bad-exit=1 bash -c 'python -m torch.distributed.run \\
    --nnodes={self.nodes} --nproc-per-node={self.gpus_per_node} --node-rank=$SLURM_NODEID \\
    --rdzv-backend=c10d --rdzv-endpoint=$MASTER_ADDR:$MASTER_PORT --rdzv-id=$SLURM_JOB_ID \\
    {self.invocation()}'
echo "finished $(date)"
"""
        return "\n".join(head) + "\n" + body

    def write(self, array: str | None = None) -> str:
        os.makedirs(self.log_dir, exist_ok=True)
        path = os.path.join(self.log_dir, f"{self.run_name}.sbatch")
        with open(path, "w") as f:
            f.write(self.sbatch_text(array))
        return path


def repetitions_needed(total_minutes: int, timeslot_minutes: int) -> int:
    """Number of consecutive allocations of ``timeslot_minutes`` that cover ``total_minutes`` (the training script
    resumes from its latest checkpoint at the start of each one)."""
    return max(1, -(-total_minutes // timeslot_minutes))


def submit(job: SlurmJob, repetitions: int, use_chain: bool, dryrun: bool) -> list[str]:
    """Job array with ``%1`` concurrency (default) or an explicit ``afterany`` chain; returns the sbatch command lines."""
    cmds = []
    if repetitions > 1 and not use_chain:
        path = job.write(array=f"0-{repetitions - 1}%1")
        cmds.append(f"sbatch {path}")
    else:
        path = job.write()
        cmds.append(f"sbatch --parsable {path}")
        for _ in range(repetitions - 1):
            cmds.append(f"sbatch --parsable --dependency=afterany:$PREV {path}")
    if dryrun:
        print(f"wrote {path}; would run:")
        for c in cmds:
            print("  " + c)
        return cmds
    prev = ""
    for c in cmds:
        out = subprocess.run(c.replace("$PREV", prev), shell=True, check=True, capture_output=True, text=True).stdout
        prev = out.strip().split(";")[0]
        print(f"submitted: {c.replace('$PREV', prev)} -> {out.strip()}")
        time.sleep(0.2)
    return cmds


def interactive(job: SlurmJob) -> str:
    opts = f"--nodes={job.nodes} --gpus-per-node={job.gpus_per_node} --time={job.time_string()} --exclusive"
    for key, val in (("partition", job.partition), ("account", job.account), ("qos", job.qos)):
        if val:
            opts += f" --{key}={val}"
    return f"salloc {opts}"


def parse_and_execute(argv=None):
    ap = argparse.ArgumentParser(description="Write and submit SLURM jobs for multi-node training runs.")
    ap.add_argument("--run_name", default="b200-debug")
    ap.add_argument("--uuid", action="store_true", help="append a short unique id to the run name")
    ap.add_argument("--python_script", default="train.py")
    ap.add_argument("--config", default=None)
    ap.add_argument("--dryrun", action="store_true", help="only write the sbatch file and print the commands")
    ap.add_argument("--interactive", action="store_true", help="print the salloc line for a debug session")
    ap.add_argument("--budget_minutes", type=int, default=120)
    ap.add_argument("--budget_hours", type=int, default=0)
    ap.add_argument("--budget_days", type=int, default=0)
    ap.add_argument("--timeslot", type=int, default=10080, help="longest single allocation in minutes")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--gpus_per_node", type=int, default=8)
    ap.add_argument("--partition", default=None)
    ap.add_argument("--account", default=None)
    ap.add_argument("--qos", default=None)
    ap.add_argument("--debug_qos", action="store_true")
    ap.add_argument("--output_dir", default=None)
    ap.add_argument("--extra_args", default="", help="extra arguments to the training script as --arg=X")
    ap.add_argument("--email", default=None)
    ap.add_argument("--repetitions", type=int, default=None)
    ap.add_argument("--custom_invocation", default=None)
    ap.add_argument("--overwrite_env", default=None, help="'VAR=X VAR2=Y'")
    ap.add_argument("--dependency", default=None)
    ap.add_argument("--disable_net_gdr", action="store_true")
    ap.add_argument("--nccl_debug", action="store_true")
    ap.add_argument("--use_chain", action="store_true", help="chain jobs with afterany instead of a job array")
    ap.add_argument("--no_rebuild", action="store_true", help="skip the kernel library build step")
    ap.add_argument("--snapshot", action="store_true",
                    help="freeze the working tree into a tar.gz, stage it to node-local storage and run from there")
    ap.add_argument("--archives", nargs="*", default=[], help="further .tar.gz files to stage on every node")
    ap.add_argument("--cast_working_dirs", action="store_true", help="the reference launcher's name for --snapshot")
    ap.add_argument("--environment", default=None,
                    help="python environment to activate in the job: a directory with bin/activate, or a packed "
                         ".tar.gz that is unpacked to node-local storage first")
    ap.add_argument("--enable_internet", action="store_true",
                    help="export the proxy given by --proxy (or $CLUSTER_PROXY) to the job")
    ap.add_argument("--proxy", default=None, help="http(s) proxy URL for --enable_internet")
    ap.add_argument("--sub_output_dir_name", default=None, help="folder under --output_dir for this run's files "
                                                                 "(default: the run name)")
    ap.add_argument("--extended_partition", action="store_true", help="submit to the 'extended' partition")
    args = ap.parse_args(argv)
    args.snapshot = args.snapshot or args.cast_working_dirs
    if args.extended_partition and not args.partition:
        args.partition = "extended"

    name = args.run_name + (f"_{secrets.token_hex(3)}" if args.uuid else "")
    total = args.budget_minutes + 60 * args.budget_hours + 24 * 60 * args.budget_days
    env = nccl_environment(args.disable_net_gdr, args.nccl_debug)
    if args.overwrite_env:
        env.update(dict(kv.split("=", 1) for kv in args.overwrite_env.split()))
    job = SlurmJob(run_name=name, python_script=args.python_script, config=args.config, extra_args=args.extra_args,
                   nodes=args.nodes, gpus_per_node=args.gpus_per_node, minutes=min(total, args.timeslot),
                   partition=args.partition, account=args.account, qos="debug" if args.debug_qos else args.qos,
                   email=args.email, output_dir=args.output_dir or os.path.join(HERE, "outputs"), env=env,
                   custom_invocation=args.custom_invocation, dependency=args.dependency,
                   rebuild_kernels=not args.no_rebuild, archives=list(args.archives), environment=args.environment,
                   proxy=(args.proxy or os.environ.get("CLUSTER_PROXY")) if args.enable_internet else None,
                   sub_dir=args.sub_output_dir_name)
    if args.snapshot:
        snap = f"{name}_code"
        path = snapshot_working_tree(os.path.join(job.output_dir, name), snap) if not args.dryrun else \
            os.path.join(job.output_dir, name, f"{snap}.tar.gz")
        job.archives.insert(0, path)
        job.run_from_snapshot = snap
    if args.interactive:
        print(interactive(job))
        return job
    reps = args.repetitions or repetitions_needed(total, args.timeslot)
    print(f"{getpass.getuser()}: {name}: {args.nodes} node(s) x {args.gpus_per_node} GPU, {total} min in {reps} job(s)")
    submit(job, reps, args.use_chain, args.dryrun)
    return job


if __name__ == "__main__":
    parse_and_execute(sys.argv[1:])
