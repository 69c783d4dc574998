from .base import (BoundCall, Segment, StepContext, Workspace, build_part, graph_safe, part_class,
                   register_part, streamed_weights_of, tensor_of, unregister_part)
from . import norm, position, attention, feed_forward, block, io  # noqa: F401  (register kinds)
from .linear import Linear

__all__ = ["BoundCall", "Segment", "StepContext", "Workspace", "build_part", "graph_safe",
           "part_class", "register_part", "streamed_weights_of", "tensor_of", "unregister_part",
           "Linear"]
