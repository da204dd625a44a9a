"""Train from the flag entry point: every config field is a ``--<field>`` flag, optionally on top of a
YAML file.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train.py \
        --config-path configs/example.yaml --tensor_model_parallel_size 2 --train_steps 100
    python examples/train.py --model_name tiny --name llama --d_model 256 --num_layers 2 --task_type synthetic \
        --vocab_size 1024 --train_steps 20 --no_save true
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ironcore_b200.config import load_trainer_config  # noqa: E402
from ironcore_b200.trainer import Trainer  # noqa: E402


def main():
    config = load_trainer_config()
    trainer = Trainer(config)
    try:
        trainer.train()
    finally:
        trainer.finalize()


if __name__ == "__main__":
    main()
