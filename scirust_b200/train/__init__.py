from .trainer import Trainer, TrainerConfig  # noqa: F401
from .schedule import WarmupCosineSchedule  # noqa: F401
