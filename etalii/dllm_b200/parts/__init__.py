from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .registry import build_part, part_factory, register_part, unregister_part  # noqa: F401
from .spec import LayerSpec, ModelSpec, ParamSpec, PartSpec, ScheduleEntry  # noqa: F401
