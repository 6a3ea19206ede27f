from .sddmm import SDDMMbase, VanillaSDDMMx86, VanillaSDDMMcuda
from .spmm import SpMMbase, VanillaSpMMx86, VanillaSpMMcuda

# the names the hot path is usually referred to by
VanillaSpMM = VanillaSpMMcuda
VanillaSDDMM = VanillaSDDMMcuda
