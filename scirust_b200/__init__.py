"""scirust_b200 - a Blackwell-native (sm_100a) deep-learning framework with the ML surface of SciRust.

Layers (top to bottom): ``cli`` -> ``models`` / ``train`` / ``generate`` -> ``nn`` -> ``autodiff`` ->
``tensor`` / ``io`` / ``data`` -> ``parallel`` -> ``ops`` (ctypes onto the native libraries in ``lib/``).
"""
__version__ = "0.1.0"
