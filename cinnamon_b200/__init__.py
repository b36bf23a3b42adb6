"""cinnamon_b200: B200-native kernels for the FP8 training path of cinnamon.

``cinnamon_b200.kernels`` is the drop-in for the reference's ``src/kernels.py``.
Importing it loads ``lib/libcinnamon_b200.so`` and raises if the library is absent.
"""
__version__ = "0.1.0"
