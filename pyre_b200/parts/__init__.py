from . import (attention, block, differential_attention, embedding, latent_attention, linear_attention, mamba2, mlp, norm,
               rotary, side_input, wkv)  # noqa: F401  (register the built-in parts)
from .base import (BoundCall, HeadGeometry, PagedKVSpec, Part, PartSpec, PositionEncoding, ProjectionLayout, StateSpec, all_graph_safe, collect_libraries, collect_tensors,
                   load_part, make_part, register_part, registered_parts)

__all__ = ["BoundCall", "HeadGeometry", "PagedKVSpec", "Part", "PartSpec", "PositionEncoding", "ProjectionLayout", "StateSpec", "collect_libraries", "collect_tensors",
           "load_part", "make_part", "register_part", "registered_parts"]
