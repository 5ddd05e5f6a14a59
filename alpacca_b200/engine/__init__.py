from .engine import CacheFull, Engine, StepEntry
from .model import DecoderModel, DecoderSpec, Run

__all__ = ["CacheFull", "Engine", "StepEntry", "DecoderModel", "DecoderSpec", "Run"]
