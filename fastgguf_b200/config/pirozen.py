"""``PirozenConfig``: the Pirozen decoder's config.json.

The class is the Python name of the host's ``PirozenConfig`` (``csrc/host/config_pirozen.cpp``): keys ``architecture``
("Pirozen"), ``vocab``, ``width``, ``norm.eps``, ``layers`` - a list whose entries give an attention mixer (sizes and
constants under ``mixer``: heads, key/value heads, key and value sizes, score scale, window, rotated dimensions and their
scaling) and a mixture of experts (``mlp``: expert size, router with its groups and identity experts, shared expert; or
null) -, an optional ``loop`` (``start``, ``stop``, ``times``: a span of layers that runs several times in a row) and an
optional ``token_side`` (``dim``: the numbers a token gives every layer from a second embedding table).
"""
from __future__ import annotations

from .base import ModelConfig


class PirozenConfig(ModelConfig):
    @classmethod
    def from_dict(cls, d: dict) -> "PirozenConfig":
        d = dict(d)
        d.setdefault("architecture", "Pirozen")
        return super().from_dict(d)
