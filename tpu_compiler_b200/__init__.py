"""B200-native execution backend for the tpu_compiler interpreter path.

``module`` mirrors ``pymlir.module`` (bindings/python/pymlir.cpp:289-311) over the
C ABI of ``libtpucb.so``; ``graphs`` builds the module text and synthetic weights
of the benchmark networks; ``calibration`` mirrors ``ActivationCalibrator``; ``pytuner.tuner``
mirrors ``pytuner.tuner`` (bindings/python/pytuner.cpp:290-310); ``cli`` is the ``tpuc-interpreter``
command line (tools/tpuc-interpreter/tpuc-interpreter.cpp).
"""
from ._lib import TpucbError, lib  # noqa: F401
from .interpreter import module  # noqa: F401
