"""B200-native decode hot path for GGUF K-quant models (Q4_K/Q6_K GEMV, Gated DeltaNet step)."""
