from .state import (CallbackHandler, DefaultFlowCallback, EarlyStoppingCallback, PrinterCallback, TrainerCallback,
                    TrainerControl, TrainerState)
from .trainer import Trainer, TrainOutput, get_last_checkpoint, set_seed
from .training_args import TrainingArguments
