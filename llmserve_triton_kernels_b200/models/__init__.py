"""Architectures as data.  Importing the package registers the built-in architecture."""

from .plan import Injection, LayerRun, LayerSpec, ModelPlan  # noqa: F401
from .model import Model  # noqa: F401
from . import kafepel, llama, nudodra, nurolorn, tenotar  # noqa: F401,E402
