"""``python train.py --config=launch_configs/<x>.yaml [--field=value ...]`` -- pretraining entry point.

Same invocation and YAML field names as the reference's train.py (train.py:1016-1076 there); launched once per GPU
by ``torchrun`` / SLURM.  Any exception still tears down the process group before the process exits.
"""
import sys

from recurrent_pretraining_b200.runtime import trainer
from recurrent_pretraining_b200.settings import parse_cli


def guarded_main() -> None:
    cfg = parse_cli(sys.argv[1:])
    try:
        trainer.main(cfg)
    except BaseException:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
        raise


if __name__ == "__main__":
    guarded_main()
