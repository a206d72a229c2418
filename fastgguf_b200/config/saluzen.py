"""``SaluzenConfig``: the Saluzen decoder's config.json.

The class is the Python name of the host's ``SaluzenConfig`` (``csrc/host/config_saluzen.cpp``): keys ``architecture``
("Saluzen"), ``vocab``, ``width``, ``norm.eps`` and ``layers`` - a list whose entries name a mixer (``type`` "parallel":
attention beside a state-space mixer; "parallel_2": chunked attention beside the gated delta rule; "latent_attention", which
may read an earlier layer's latents through ``kv_from``; sizes and constants under ``mixer``) and a dense feed-forward
(``mlp``, or null).
"""
from __future__ import annotations

from .base import ModelConfig


class SaluzenConfig(ModelConfig):
    @classmethod
    def from_dict(cls, d: dict) -> "SaluzenConfig":
        d = dict(d)
        d.setdefault("architecture", "Saluzen")
        return super().from_dict(d)
