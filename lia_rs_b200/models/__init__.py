from .decoder import DecoderModel, ModelSpec, ScheduleEntry
from . import minicpm5_llama, nafevik, vatunex, zipelix, pilutar  # noqa: F401  (register the architectures)

__all__ = ["DecoderModel", "ModelSpec", "ScheduleEntry"]
