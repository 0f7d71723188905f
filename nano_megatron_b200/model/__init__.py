"""Import-path alias: the reference keeps its sharded models under ``nano_megatron.model``
(nano_megatron/model/__init__.py:1-22); here the package is :mod:`nano_megatron_b200.models`.
``nano_megatron_b200.model``, ``.model.tp_gpt`` and ``.model.pipeline`` resolve to the same
module objects, so code written against the reference's paths keeps working."""
import sys as _sys

from .. import models as _models
from ..models import pipeline, tp_gpt
from ..models import *  # noqa: F401,F403

__all__ = list(_models.__all__)
_sys.modules[__name__ + ".tp_gpt"] = tp_gpt
_sys.modules[__name__ + ".pipeline"] = pipeline
