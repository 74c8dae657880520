"""The model, the step function, the generation loop and trace replay."""

from .generate import (COMPLETE, DECODING, EXHAUSTED, PREFILLING, Ending, plan_batches,
                       plan_prefill)
from .model import DecoderModel
from .step import StepContext, StepStager
from .engine import Engine

__all__ = ["COMPLETE", "DECODING", "EXHAUSTED", "PREFILLING", "Ending", "plan_batches",
           "plan_prefill", "DecoderModel", "StepContext", "StepStager", "Engine"]
