"""Checkpoint conversion between Hugging Face Llama models and the framework's flat parameter files."""
