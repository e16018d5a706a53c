"""Counterpart of ``amct_pytorch/experimental/quantization/DeepSeekV3.2`` (a script directory in the reference;
a package here because a dot is not valid in a module name).  ``deploy`` holds the offline checkpoint export."""
