"""The reference's ``dae`` Python API over the B200 runtime.

Put the directory that holds this package on ``sys.path`` (``PYTHONPATH=<repo>/vdcores_b200``) and
model scripts written against the reference (``from dae.launcher import *``, ``from dae.schedule
import *``, ``from dae.model import *``, ``from dae.util import *``) import unchanged: same class
names, constructor arguments and instruction encodings (reference python/dae/*.py), while
``dae.runtime`` is the ctypes binding of libvdcores_b200.so instead of the compiled sm_90a extension.
"""
from . import launcher
from . import util

__all__ = ["launcher", "util"]
