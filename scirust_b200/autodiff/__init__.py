from .tape import Tape, Var, TapeError  # noqa: F401
from .optim import Sgd, Adam, AdamW, Optimizer, MuonOptimizer, TrainOptimizer  # noqa: F401
from .scheduler import (LrSchedule, Constant, StepDecay, Exponential, CosineAnnealing, WarmupCosine,  # noqa: F401
                        ReduceOnPlateau)
from .nd import NdTape, NdVar, NdTapeError  # noqa: F401
