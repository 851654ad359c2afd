from .fsdp import FSDPConfig, FSDPTrainingBackend
from .native import NativeTrainingBackend, warmup_cosine
from .protocol import TrainingBackend
from .pytorch import PyTorchTrainingBackend
from .stubs import JAXTrainingBackend, TorchaxTrainingBackend
from .tensor_parallel import TensorParallelTrainingBackend
from .torch_func import TorchFuncTrainingBackend
from .pytorch_factory import (create_adamw_optimizer, create_backend_with_scheduler, create_cross_entropy_loss,
                              create_pytorch_backend, create_warmup_cosine_scheduler, load_model_weights, parse_dtype)

__all__ = ["FSDPConfig", "FSDPTrainingBackend", "NativeTrainingBackend", "warmup_cosine", "TrainingBackend",
           "PyTorchTrainingBackend", "TorchFuncTrainingBackend", "TensorParallelTrainingBackend", "JAXTrainingBackend", "TorchaxTrainingBackend", "create_adamw_optimizer", "create_backend_with_scheduler",
           "create_cross_entropy_loss", "create_pytorch_backend", "create_warmup_cosine_scheduler",
           "load_model_weights", "parse_dtype"]
