"""Block arrangements and the parts at the two ends of the model.

``PreNorm``: x += mixer(norm1(x)); x += feed_forward(norm2(x)) -- the residual placement
of the reference's forward (src/locus/model/llama.cpp:485-509).  The residual stream x is
float32 in every mode; the normed activations have the model's element type.

``Embedding``: x = table[token] (llama.cpp:450).  ``LmHead``: logits = W . h in float32,
W being the embedding table when the head is tied (llama.cpp:292-297, 512-513): the head then
names the embedding's tensor as the source of its weight.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import (Arrangement, Part, PartSpec, TensorSource, make_part, register_arrangement,
                   register_embedding, register_head)


class PreNorm(Arrangement):
    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec,
                 feed_forward: PartSpec, mixer_prefix: str = "self_attn", ff_prefix: str = "mlp",
                 norm1_name: str = "input_layernorm", norm2_name: str = "post_attention_layernorm") -> None:
        super().__init__(prefix)
        self.hidden = hidden
        self.norm1 = make_part("norm", norm, f"{prefix}.{norm1_name}")
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.norm2 = make_part("norm", norm, f"{prefix}.{norm2_name}")
        self.ff = make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")

    takes_pending_add = True

    def sub_parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ff]

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        self.norm1.forward(x, h, add=rt.take_pending())
        self.mixer.forward(h, batch, cache, x, rt)
        self.norm2.forward(x, h)
        self.ff.forward(h, batch, x, rt)


class Embedding(Part):
    def __init__(self, prefix: str, *, vocab: int, hidden: int) -> None:
        super().__init__(prefix)
        self.vocab, self.hidden = int(vocab), int(hidden)

    def param_shapes(self):
        return {"table": (self.vocab, self.hidden)}

    def sources(self):
        return [TensorSource(self.prefix + ".weight", (self.vocab, self.hidden), "table")]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, tokens: torch.Tensor, out: torch.Tensor) -> None:
        K.embed_rows(tokens, self.params["table"], out)


class LmHead(Part):
    """``tied_to``: the checkpoint tensor that is the head's weight when the head has none of its own
    (the embedding table of a tied model); two parts that name the same tensor share one device copy."""

    def __init__(self, prefix: str, *, vocab: int, hidden: int, tied_to: str = "") -> None:
        super().__init__(prefix)
        self.vocab, self.hidden, self.tied_to = int(vocab), int(hidden), str(tied_to or "")

    def param_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def sources(self):
        return [TensorSource(self.tied_to or self.prefix + ".weight", (self.vocab, self.hidden), "weight")]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def forward(self, h: torch.Tensor, logits: torch.Tensor) -> None:
        K.linear(h, self.params["weight"], logits)


register_arrangement("pre_norm", PreNorm)
register_embedding("embedding", Embedding)
register_head("linear", LmHead)
