"""A small, whole inference engine for the Qwen2 dense decoder on one B200 (sm_100a)."""

from . import models, parts  # noqa: F401  (fills the registries)

__version__ = "0.1.0"
