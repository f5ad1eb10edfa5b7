"""Parallel runtime: process groups, symmetric (peer-mapped) memory, fused collectives,
data/tensor parallel layers, logical device meshes, and the host-side fixed-order collectives."""


def __getattr__(name):
    """Lazy exports (the device-side modules load the CUDA library when they are imported)."""
    if name == "make_grad_reducer":
        from .data_parallel import make_grad_reducer
        return make_grad_reducer
    if name == "FlatDataParallel":
        from .ddp import FlatDataParallel
        return FlatDataParallel
    if name == "PipelineModel":
        from .pipeline import PipelineModel
        return PipelineModel
    if name == "InterleavedPipelineModel":
        from .pipeline import InterleavedPipelineModel
        return InterleavedPipelineModel
    if name == "ring_attention":
        from .context_parallel import ring_attention
        return ring_attention
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
