"""GPT-2 / GPT-3 / MoE trainer with the flag surface of the reference's ``train_gpt2cu``:

    python -m llm_kittens_b200.cli.train_gpt2cu -e d12 -i "data/train_*.bin" -j "data/val_*.bin" \
        -b 64 -t 1024 -d 524288 -l 6e-4 -u 700 -q 0 -c 0.1 -z 1 -o log124M
    torchrun --nproc-per-node 8 -m llm_kittens_b200.cli.train_gpt2cu ...     (one process per GPU)
"""
import sys

from .train import run


def main() -> int:
    return run(sys.argv[1:], "gpt2")


if __name__ == "__main__":
    sys.exit(main())
