"""Drop-in module: `import flash_attn_v100` resolves to the sm_100a library's
operator API (same function names and positional signatures as the reference's
pybind module, flash_attn.cpp:224-255)."""
from flash_attn_v100_b200.ops import *  # noqa: F401,F403
from flash_attn_v100_b200.ops import REFERENCE_EXPORTS as __all__  # noqa: F401
