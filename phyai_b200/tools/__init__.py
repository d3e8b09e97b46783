"""Pre/post-processing tools that sit around the engines (the reference ships them as ``phyai-utils-tools``)."""

from . import processing, tokenizer  # noqa: F401
from .processing import BaseModelProcessor, ProcessorPipeline, ProcessorStep, ProcessorStepRegistry  # noqa: F401

__version__ = "0.1.0"

__all__ = ["__version__", "processing", "tokenizer", "BaseModelProcessor", "ProcessorPipeline", "ProcessorStep", "ProcessorStepRegistry"]
