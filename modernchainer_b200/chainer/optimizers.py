"""Optimizers (`chainer.optimizers.*`), python/chainer/optimizers.py of the reference."""
from . import SGD, Adam, AdamW, LinearWarmupCosineLR, MomentumSGD

__all__ = ["Adam", "AdamW", "LinearWarmupCosineLR", "MomentumSGD", "SGD"]
