"""B200-native GRPO loss boundary (placeholder until the CUDA library is wired in)."""
