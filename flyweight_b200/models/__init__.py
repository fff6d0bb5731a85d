from . import diforax, fobatar, gukosun, kemitar, lfm2  # noqa: F401  (register the architectures)
from .diforax import DiforaxForCausalLM
from .fobatar import FobatarForCausalLM
from .gukosun import GukosunForCausalLM
from .kemitar import KemitarForCausalLM
from .lfm2 import Lfm2ForCausalLM

__all__ = ["DiforaxForCausalLM", "FobatarForCausalLM", "GukosunForCausalLM", "KemitarForCausalLM", "Lfm2ForCausalLM"]
