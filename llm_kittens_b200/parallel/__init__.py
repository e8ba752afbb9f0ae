"""Multi-GPU machinery: ZeRO sharding plans, process-group bootstrap, library and fused communication."""
