"""Links and modules (`L.*`), python/chainer/links.py of the reference."""
from . import BatchNorm, Conv2d, ConvTranspose2d, Embedding, LayerNorm, Linear, MultiHeadAttention, RMSNorm

__all__ = ["BatchNorm", "Conv2d", "ConvTranspose2d", "Embedding", "LayerNorm", "Linear", "MultiHeadAttention", "RMSNorm"]
