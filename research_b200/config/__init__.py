"""Config protocols, base config pieces and the file loader (rollouts/config/__init__.py)."""

from .base import (PROVIDER_DEFAULTS, BaseEnvironmentConfig, BaseEvaluationConfig, BaseModelConfig, BaseOutputConfig,
                   infer_provider_from_model)
from .loader import load_config_from_file, validate_config_protocol
from .protocols import PROTOCOLS, HasEnvironmentConfig, HasEvaluationConfig, HasModelConfig, HasOutputConfig

__all__ = ["HasModelConfig", "HasEnvironmentConfig", "HasEvaluationConfig", "HasOutputConfig", "PROTOCOLS",
           "BaseModelConfig", "BaseEnvironmentConfig", "BaseEvaluationConfig", "BaseOutputConfig", "PROVIDER_DEFAULTS",
           "infer_provider_from_model", "load_config_from_file", "validate_config_protocol"]
