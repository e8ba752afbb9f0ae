"""llm_kittens_b200: a B200-native (sm_100a) LLM pre-training framework.

PyTorch is the framework layer (tensors, streams, torch.distributed bootstrap); every hot op is a
hand-written CUDA kernel from ``csrc/`` loaded through ctypes (``ops/``); models run explicit
forward/backward schedules over flat parameter / gradient / activation arenas (``models/``,
``runtime/``); ZeRO sharding and the fused collective kernels live in ``parallel/``; file formats,
schedulers, logging and the data loaders in ``utils/``; command-line trainers in ``cli/``.
"""
__version__ = "0.1.0"
