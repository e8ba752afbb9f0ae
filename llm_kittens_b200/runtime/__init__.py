"""Training runtime: optimizer state, step orchestration, checkpointing, evaluation, sampling."""
