"""Model families (GPT-2/3, Llama-3, MoE) over flat parameter buffers with explicit fwd/bwd schedules."""
