from .sddmm import SDDMMbase, VanillaSDDMMx86, VanillaSDDMMcuda
from .spmm import SpMMbase, VanillaSpMMx86, VanillaSpMMcuda

# the names the hot path is usually referred to by
VanillaSpMM = VanillaSpMMcuda
VanillaSDDMM = VanillaSDDMMcuda

# SpMM followed by SDDMM on its output, in one pass (no counterpart class in the reference: it runs the two
# modules above back to back)
from .fused import AggregateThenScore
