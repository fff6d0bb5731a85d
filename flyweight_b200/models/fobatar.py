"""Fobatar: registration of the architecture name with its configuration and model.  The model is the generic
``DecoderModel`` over ``FobatarConfig.model_spec()``: layers in the sandwich arrangement (a norm on both sides
of every sublayer, one constant on what they add), attention inside chunks with convolutions on q, k, v, a
zero sink and a gate per head, or attention over a cached latent with a gate per head, experts chosen by the
token's id beside a shared expert, a stretch of layers that may run several times, a final norm and the
embedding table as the head."""
from __future__ import annotations

from ..config.fobatar import FobatarConfig
from ..config.registry import register_architecture
from ..parts.base import Precision
from ..parts.model import DecoderModel


class FobatarForCausalLM(DecoderModel):
    config_class = FobatarConfig

    def __init__(self, config: FobatarConfig, precision: Precision, device):
        self.config = config
        super().__init__(config.model_spec(), precision, device)


register_architecture("Fobatar", FobatarConfig, FobatarForCausalLM)
