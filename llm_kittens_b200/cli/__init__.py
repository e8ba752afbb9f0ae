"""Command-line trainers: ``python -m llm_kittens_b200.cli.train_gpt2cu`` / ``train_llama3cu``."""
