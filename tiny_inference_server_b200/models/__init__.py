"""Registered architectures."""
from .base import Model, ScheduleEntry, StepOutput
from . import gqa_mtp  # noqa: F401  (registers "gqa_mtp_transformer")
from . import kefisun  # noqa: F401  (registers "Kefisun")
from . import mizidra  # noqa: F401  (registers "Mizidra")
from . import biruvik  # noqa: F401  (registers "Biruvik")
from . import kubolorn  # noqa: F401  (registers "Kubolorn")

__all__ = ["Model", "ScheduleEntry", "StepOutput"]
