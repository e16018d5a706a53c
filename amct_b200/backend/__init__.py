"""Bridge between torch tensors and the C-ABI CUDA library."""
