from .llama import ConfigError, LlamaConfig  # noqa: F401
from .nurolorn import NurolornConfig  # noqa: F401
from .kafepel import KafepelConfig  # noqa: F401
from .nudodra import NudodraConfig  # noqa: F401
from .tenotar import TenotarConfig  # noqa: F401
from .registry import (  # noqa: F401
    Architecture,
    architecture_of,
    get_architecture,
    known_architectures,
    read_config,
    register_architecture,
    unregister_architecture,
)
