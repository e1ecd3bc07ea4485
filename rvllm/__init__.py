"""`import rvllm`: the reference's package name for this engine's entry points.

The reference's Python package is called `rvllm` and is expected to expose `Sampler`,
`Tokenizer` and `__version__ == "0.1.0"` (tests/test_rvllm_python.py:1-5 of the reference).
Everything lives in `rvllm_b200`; this module only re-exports it.
"""
from rvllm_b200 import *            # noqa: F401,F403
from rvllm_b200 import __all__, __version__  # noqa: F401
