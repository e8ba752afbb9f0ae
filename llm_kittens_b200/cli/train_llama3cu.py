"""Llama-3 trainer with the flag surface of the reference's ``train_llama3cu`` (default ``-x 0``: a
host-only dry run that validates the descriptor / checkpoint header and the ZeRO layout):

    python -m llm_kittens_b200.cli.train_llama3cu -e llama3:8B -z 3 -pn 8 -x 0
    torchrun --nproc-per-node 8 -m llm_kittens_b200.cli.train_llama3cu -e llama3.2:1B -z 2 -b 8 -t 2048 -x 100 ...
"""
import sys

from .train import run


def main() -> int:
    return run(sys.argv[1:], "llama3")


if __name__ == "__main__":
    sys.exit(main())
