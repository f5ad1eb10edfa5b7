from .trainer import Trainer, TrainerConfig  # noqa: F401
from .schedule import ConstantSchedule, WarmupCosineSchedule  # noqa: F401
