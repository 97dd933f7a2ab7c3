from .loader import ConfigError, GlobalConfig, batch_triple, expand_operator_types
from .schema import FIELDS, GROUPS, OPERATOR_CHOICES, SUPPORTED_OPERATORS

__all__ = ["GlobalConfig", "ConfigError", "FIELDS", "GROUPS", "OPERATOR_CHOICES", "SUPPORTED_OPERATORS",
           "batch_triple", "expand_operator_types"]
