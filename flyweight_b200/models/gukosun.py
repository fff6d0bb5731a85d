"""Gukosun: registration of the architecture name with its configuration and model.  The model is the
generic ``DecoderModel`` over ``GukosunConfig.model_spec()``: layers in the parallel arrangement (one norm,
mixer and feed-forward side by side, a scale per channel on each, a token-indexed side input behind them),
windowed attention with a sink, mixed values and an output gate, or an attention beside a decayed linear
attention as mixer, a dense feed-forward, a final norm, an untied head and scaled logits."""
from __future__ import annotations

from ..config.gukosun import GukosunConfig
from ..config.registry import register_architecture
from ..parts.base import Precision
from ..parts.model import DecoderModel


class GukosunForCausalLM(DecoderModel):
    config_class = GukosunConfig

    def __init__(self, config: GukosunConfig, precision: Precision, device):
        self.config = config
        super().__init__(config.model_spec(), precision, device)


register_architecture("Gukosun", GukosunConfig, GukosunForCausalLM)
