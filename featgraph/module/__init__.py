from featgraph_b200.module import (SDDMMbase, SpMMbase, VanillaSDDMM, VanillaSDDMMcuda,  # noqa: F401
                                   VanillaSDDMMx86, VanillaSpMM, VanillaSpMMcuda, VanillaSpMMx86)
