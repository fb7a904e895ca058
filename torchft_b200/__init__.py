"""torchft_b200: per-step fault tolerance for PyTorch training, built natively for B200."""
