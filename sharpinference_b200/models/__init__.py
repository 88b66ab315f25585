"""Model assembly: the generic decoder and the architectures built on it."""
from .model import DecoderModel, ScheduleEntry

__all__ = ["DecoderModel", "ScheduleEntry"]
