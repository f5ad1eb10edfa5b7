"""scirust_b200 - a Blackwell-native (sm_100a) deep-learning framework with the ML surface of SciRust.

Layers (top to bottom): ``cli`` -> ``models`` / ``train`` / ``generate`` -> ``nn`` -> ``autodiff`` ->
``tensor`` / ``io`` / ``data`` -> ``parallel`` -> ``ops`` (ctypes onto the native libraries in ``lib/``).

Beside that stack (imported on demand, nothing here is loaded at package import):
``compute`` (contracts, capability profiles, topology, autotuner) - ``canonical`` (tensor IR, planner, fusion) - ``numerics``
(exact accumulation, portable math, low precision, search over representations) - ``quantization`` / ``quantization_methods``
- assurance: ``certify``, ``verify``, ``conformal``, ``calibration``, ``privacy``, ``xai``, ``pruning`` - science and classical
ML on batched tensors: ``dsp``, ``fixed``, ``geometry``, ``quantum`` / ``vqnet``, ``physics``, ``ode``, ``symbolic``, ``einsum``,
``interp``, ``stats``, ``learning``, ``causal``, ``sequential``, ``estimation``, ``monitoring``, ``retrieval``, ``nlp`` - tooling:
``aot``, ``homomorphic``, ``automl``, ``mlops``, ``search``, ``embed``, ``sparse``, ``fusion``, ``cpu_kernels``.
"""
__version__ = "0.1.0"
