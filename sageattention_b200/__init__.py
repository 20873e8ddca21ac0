"""B200-native (sm_100a) NVFP4 flash attention behind the ``sageattention.nvfp4`` API.

``sageattention_b200.nvfp4`` mirrors the public names of the reference package
``sageattention.nvfp4`` (thad0ctor/SageAttention); the compute lives in hand-written CUDA reached
through a plain C ABI (``include/nvfp4_b200.h``).  There is no CPU or Triton fallback: importing
works anywhere, calling an operator without the built library raises.
"""

__version__ = "0.1.0"
