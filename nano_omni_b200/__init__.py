"""B200 (sm_100a) kernels for the MiniMax-H3 DiT attention path of nano-omni.

The package mirrors the reference's Kernel plug-in interface (``core``) and binds
each kernel class to an entry point of ``libnano_omni_b200.so`` (``_lib``).
"""

from nano_omni_b200.core import Arguments, Config, DType, Kernel, MmaType, ScratchLayout, TensorDesc, Workload

__all__ = ["Arguments", "Config", "DType", "Kernel", "MmaType", "ScratchLayout", "TensorDesc", "Workload"]
