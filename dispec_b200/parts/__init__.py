"""Built-in parts; importing this package registers them."""
from dispec_b200.parts import (attention, block, clamped_glu, embedding, latent_attention,  # noqa: F401
                                linear_attention, moe, norms, rotary, swiglu, xielu)
from dispec_b200.parts.base import (Block, CacheNeed, CacheTensor, FeedForward, Mixer, Norm, Part, PartSpec,
                                    PositionEncoding, StateNeed, TensorSpec, WideStream)

__all__ = ["Block", "CacheNeed", "CacheTensor", "FeedForward", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "StateNeed", "TensorSpec", "WideStream"]
