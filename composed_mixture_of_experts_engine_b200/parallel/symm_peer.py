"""Peer-memory (NVLink P2P) transport for the expert-parallel MoE: placeholder until the kernels are bound."""

from __future__ import annotations


def available(topology, axis: str) -> bool:
    return False
