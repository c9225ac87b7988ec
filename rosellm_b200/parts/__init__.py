from .base import (
    KVCacheSpec,
    ParamSpec,
    Part,
    StateSpec,
    build_part,
    part_class,
    register_part,
    unregister_part,
)
from .spec import Concat, LayerSpec, ModelSpec, PartSpec, RunEntry

__all__ = [
    "Concat",
    "KVCacheSpec",
    "LayerSpec",
    "ModelSpec",
    "ParamSpec",
    "Part",
    "PartSpec",
    "RunEntry",
    "StateSpec",
    "build_part",
    "part_class",
    "register_part",
    "unregister_part",
]
