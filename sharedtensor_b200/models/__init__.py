from .char_rnn import CharRNN, flat_gradient, flatten_parameters
from .gpt2 import GPT2, GPT2Config

__all__ = ["CharRNN", "GPT2", "GPT2Config", "flatten_parameters", "flat_gradient"]
