"""supergrok15_b200: a Blackwell-native (sm_100a) grokking-optimizer framework.

Public surface: the eleven ``torch.optim`` optimizers and their meta-networks (``optim``), the model zoo
(``models``), the native-kernel wrappers (``ops``), ZeRO-sharded data parallelism with in-kernel
collectives (``parallel``), the race driver (``race``) and utilities (``utils``).
The package name drops the dot of "SuperGrok1.5" because a Python package name cannot contain one;
``grokking_optimizers`` is a drop-in alias exposing the reference's import paths.
"""
from . import _build
from .optim import *  # noqa: F401,F403
from .optim import __all__ as _optim_all

__version__ = "0.1.0"
__all__ = list(_optim_all) + ["native_available"]


def native_available() -> bool:
    return _build.native_available()
