"""Step engines: the CUDA-graph captured training step of a whole model
(:class:`Trainer`) and of a pipeline stage under the 1F1B schedule
(:class:`PipelineTrainer`)."""
from .pipeline_trainer import PipelineTrainer
from .trainer import Trainer

__all__ = ["PipelineTrainer", "Trainer"]
