"""Mamba-2 SSD ops of the INT8 prefill path (module and function names of ``linquant/kernels/mamba2``)."""
