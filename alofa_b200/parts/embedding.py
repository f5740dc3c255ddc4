"""Token embedding and the output head.

``h[r] = embed[id_r]`` with ids outside the vocabulary refused
(src/alofa/model/arch/qwen.mojo:1391-1413); with ``scale`` the row is
multiplied by it, and with ``sinusoid_base`` a position vector is added whose
entry 2i is ``sin(p * base^(-2i/hidden))`` and entry 2i + 1 the cosine of the
same angle (frequencies made in float64 and rounded to fp32 once, the angle an
fp32 product, precise sine and cosine).  The head multiplies the normed
rows whose logits are wanted by ``lm_head.weight`` if the file has it, else by
the embedding when the two are tied (qwen.mojo:1077-1089, 1512-1523); a tied
head shares the embedding's memory.  With ``scale`` the logits are multiplied
by it; with ``softcap`` they are then bounded by ``softcap * tanh(logits /
softcap)``."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, register_part
from .linear import STORE, Linear


class TokenEmbedding(Part):
    family = "embedding"
    graph_safe = True
    reads_fed_tokens = True  # honours ctx.token_src: a step may be launched before the host has seen its tokens

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.name = self.prefix + str(self.params.get("weight_name", "weight"))
        self.weight = None
        self.scale = self.params.get("scale")
        self.sinusoid_base = self.params.get("sinusoid_base")
        self.freq = None

    def tensors(self):
        return {self.name: TensorSpec((self.vocab, self.hidden))}

    def load(self, state):
        self.weight = state[self.name]
        if self.sinusoid_base is not None:
            i = torch.arange((self.hidden + 1) // 2, dtype=torch.float64)
            self.freq = (float(self.sinusoid_base) ** (-2.0 * i / self.hidden)).to(torch.float32).to(self.weight.device)

    def forward(self, ctx, h):
        fed = ctx.fed_tokens is not None
        if self.scale is not None or self.freq is not None:
            ops.embed_scaled(h, self.weight, ctx.token_ids, ctx.positions, 1.0 if self.scale is None else float(self.scale), self.freq, ctx.status,
                             ctx.token_src if fed else None, ctx.fed_tokens)
            return
        ops.embed_gather(h, self.weight, ctx.token_ids, ctx.status, ctx.token_src if ctx.fed_tokens is not None else None, ctx.fed_tokens)

class LinearHead(Part):
    family = "head"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.tied_to = self.params.get("tied_to")
        self.name = self.prefix + str(self.params.get("weight_name", "weight"))
        self.scale = self.params.get("scale")  # the logits are multiplied by this (None: by nothing)
        self.softcap = self.params.get("softcap")  # then bounded: softcap * tanh(logits / softcap) (None: not)
        if self.softcap is not None and not float(self.softcap) > 0:
            raise AlofaError("invalid_argument", "a head's softcap must be positive", f"softcap={self.softcap}")
        self.linear = None

    def tensors(self):
        if self.tied_to is not None and self.tied_to == self.name:
            return {}  # the embedding's own tensor, which the embedding lists
        return {self.name: TensorSpec((self.vocab, self.hidden), optional=self.tied_to is not None)}

    def load(self, state):
        name = self.name
        if name in state:
            weight = state[name]
        elif self.tied_to is not None and self.tied_to in state:
            weight = state[self.tied_to]
        else:
            raise AlofaError("invalid_argument", "the model has no output head weight", f"name={name} tied_to={self.tied_to}")
        self.linear = Linear(weight, None, STORE)

    def forward(self, ctx, x):
        logits = ctx.buf((x.shape[0], self.vocab), torch.float32)
        self.linear(logits, x, buf=ctx.buf)
        if self.scale is not None and float(self.scale) != 1.0:
            ops.scale_rows(logits, float(self.scale))
        if self.softcap is not None:
            ops.softcap_rows(logits, float(self.softcap))
        return logits

register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
