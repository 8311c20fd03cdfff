"""The arrangement of a layer's parts. ``pre_norm``: h += mixer(norm1(h)); h += feed_forward(norm2(h))
(src/Starlings.Roost.Models.Tiny/RoostTiny.cs:40,49-50,54). The residual stream is carried beside the branch
output so that each residual sum is fused into the norm that follows it; the stream is stored in the
activation dtype and every sum is formed in 32-bit and rounded once."""
from __future__ import annotations

import torch

from ..config.spec import BlockSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, Block, Runtime, register_block


class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)

    def sub_parts(self):
        return {"input_norm": self.input_norm, "mixer": self.mixer, "post_mixer_norm": self.post_mixer_norm,
                "feed_forward": self.feed_forward}

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        return {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer),
                "post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward)}

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        """``h`` is the previous branch output (or the embedding), ``residual`` the stream before it was added
        (None at the first block). Returns the feed-forward's output and the stream it is still to be added to."""
        if residual is None:
            residual = h
            x = self.input_norm(h)
        else:
            x, residual = self.input_norm.add_norm(h, residual)
        a = self.mixer(x, batch, cache, write_cache)
        y, residual = self.post_mixer_norm.add_norm(a, residual)
        return self.feed_forward(y, batch), residual


class PreNormWideBlock(Block):
    """The same arrangement over a stream that is kept and summed in 32-bit whatever the activation dtype is: the
    embedding hands over a float32 stream, every norm reads it (adding the branch output before it first, in 32-bit)
    and writes the activation dtype. The feed-forward and its norm may be absent."""

    def __init__(self, spec: BlockSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.feed_forward = self.post_mixer_norm = None
        if spec.feed_forward is not None:
            if spec.post_mixer_norm is None:
                raise ValueError("pre_norm_wide: a feed-forward needs the norm before it")
            self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)

    def sub_parts(self):
        parts = {"input_norm": self.input_norm, "mixer": self.mixer}
        if self.feed_forward is not None:
            parts.update({"post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward})
        return parts

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        subs = {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer)}
        if spec.feed_forward is not None:
            subs.update({"post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward)})
        return subs

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        if residual is None:
            if h.dtype != torch.float32:
                raise ValueError("pre_norm_wide: the embedding must hand over a float32 stream")
            residual = h
            x = self.input_norm(h)
        else:
            x, residual = self.input_norm.add_norm(h, residual)
        a = self.mixer(x, batch, cache, write_cache)
        if self.feed_forward is None:
            return a, residual
        y, residual = self.post_mixer_norm.add_norm(a, residual)
        return self.feed_forward(y, batch), residual


register_block("pre_norm", PreNormBlock)
register_block("pre_norm_wide", PreNormWideBlock)
