"""Importable name of the engine.

The sources live in the folder ``vllm-from-scratch_b200`` next to this one; a
hyphen cannot appear in a Python module name, so this package only points its
search path at that folder and re-exports the public interface found there.
"""

from pathlib import Path as _Path

__path__.insert(0, str(_Path(__file__).resolve().parent.parent / "vllm-from-scratch_b200"))

from .api import *  # noqa: E402,F401,F403
from .api import __all__  # noqa: E402,F401
