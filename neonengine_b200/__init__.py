"""B200-native gpt-oss-shaped MoE layer: CUDA kernels behind the ``libneon_moe`` C ABI."""
