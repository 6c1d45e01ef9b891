"""CPU oracle of the RL-Spline-KV feature path.  Test infrastructure, not product code:
only ``tests/``, the smoke entry and the benchmark's CPU-baseline leg may import it."""
