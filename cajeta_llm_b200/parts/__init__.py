"""Parts a layer is put together from; importing the package registers the built-in ones."""
from .base import (KvNeed, Part, Runtime, StateNeed, make_part, register_part, registered_parts,  # noqa: F401
                   unregister_part)
from .plan import LayerSpec, ModelPlan, ParamSpec, PartSpec, ScheduleEntry  # noqa: F401
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registration)
