"""Model zoo: Llama 3.x, Qwen3 dense / MoE, Qwen3.5 hybrids, LFM2, MNIST."""
