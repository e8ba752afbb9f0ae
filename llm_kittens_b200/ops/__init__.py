"""Python wrappers of the hand-written sm_100a kernels (one module per op family)."""
