"""Layer parts: norms, position encodings, mixers, feed-forwards, their arrangement in a block,
embedding and head.  Each takes its sizes and constants as parameters and is chosen by name from
a registry; see ``registry`` for the interface of each family."""
from .registry import FAMILIES, TensorDecl, get_part, part, register_part  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
