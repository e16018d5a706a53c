"""Mirrors of the reference's ``amct_pytorch/experimental`` scripts that sit either side of the quantized Linear."""
