from . import gpt2  # registers GPT2LMHeadModel
from .model import Layer, Model, named_params_of_spec

__all__ = ["Layer", "Model", "named_params_of_spec", "gpt2"]
