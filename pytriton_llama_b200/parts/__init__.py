"""Parts of a decoder layer.  Importing this package registers the built-in kinds."""
from .base import (CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, part_kinds,  # noqa: F401
                   register_part)
from . import attention, block, rmsnorm, rope, swiglu  # noqa: F401
