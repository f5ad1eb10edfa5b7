from .logging import TrainingLogger, TensorBoardWriter, read_tfrecords, crc32c  # noqa: F401
from .profiling import nvtx_range, DeviceTimer, annotate_model  # noqa: F401
from .planning import plan, n_params, MemoryPlan  # noqa: F401
