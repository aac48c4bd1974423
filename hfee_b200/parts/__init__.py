from .base import CATEGORIES, Block, Mixer, Part, Runtime, build_part, part_class, register_part
from . import (attention, block, conv, delta_rule, distance_attention, embedding, gated_attention, gated_linear_attention,
               latent_attention, linear_attention, merge, mlp, moe, norm, parallel, recurrent, rotary, sigmoid_attention,
               softmax_attention)  # noqa: F401  (register the built-in kinds)
from .model import DecoderModel, model_tensor_needs

__all__ = ["CATEGORIES", "Mixer", "Part", "Runtime", "build_part", "part_class", "register_part",
           "DecoderModel", "model_tensor_needs"]
