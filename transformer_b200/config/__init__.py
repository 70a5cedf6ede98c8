from .llama import LlamaMeta
from .registry import (Architecture, ConfigError, architecture_for, register_architecture,
                       registered_architectures, unregister_architecture)
