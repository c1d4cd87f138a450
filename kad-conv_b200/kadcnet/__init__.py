"""KAD-CNet-S for B200: module definitions (kadcnet.model), their CUDA execution (kadcnet.engine),
post-processing (kadcnet.postprocess) and the inference entry point (kadcnet.runtime.load_model)."""
from .model import DetectionModel
from .pipeline import DetectionPipeline
from . import preprocess
from .runtime import StaticGraph, load_model

__all__ = ['DetectionModel', 'load_model', 'StaticGraph', 'DetectionPipeline']
