"""Drop-in call surface of ``linquant.kernels`` (zoo chunk ops, Mamba-2 SSD ops, Hadamard prologue)."""
