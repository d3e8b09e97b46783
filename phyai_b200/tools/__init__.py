"""Pre/post-processing tools that sit around the engines (the reference ships them as ``phyai-utils-tools``)."""

from . import processing, tokenizer  # noqa: F401
from .processing import ProcessorPipeline, ProcessorStep, ProcessorStepRegistry  # noqa: F401

__all__ = ["processing", "tokenizer", "ProcessorPipeline", "ProcessorStep", "ProcessorStepRegistry"]
