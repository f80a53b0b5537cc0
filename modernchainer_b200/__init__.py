"""modernchainer_b200: Python binding of the sm_100a training-step backend.

The package mirrors the reference's Python surface (`chainer.Variable`, `F.*`, `O.Adam`,
`GradScaler`; python/chainer/*.py and crates/modern-chainer-python/src/lib.rs in the
reference) on top of the C ABI declared in include/mcb.h.  All arithmetic runs in
libmcb.so on the GPU; importing the package works without a GPU, creating a Context
does not.
"""
from . import _lib
from .api import (BF16, F16, F32, I32, I64, U8, SGD, Adam, AdamW, Arena, ConstantLR, Context, DeviceArray, F, GradScaler,
                  LinearWarmupCosineLR, McbError, Model, MomentumSGD, PolynomialLR, StaticStep, StepLR, Variable, autocast, bf16_bits_to_f32,
                  clip_grad_norm, device_count, f32_to_bf16_bits, load_checkpoint, no_grad, ops, save_checkpoint, zero_grad)

__all__ = ["Context", "DeviceArray", "Variable", "F", "StaticStep", "Adam", "AdamW", "SGD", "MomentumSGD", "GradScaler", "Model", "Arena",
           "McbError", "ops", "no_grad", "autocast", "zero_grad", "clip_grad_norm", "save_checkpoint", "load_checkpoint", "LinearWarmupCosineLR", "StepLR",
           "ConstantLR", "PolynomialLR", "device_count", "F32", "I64", "I32", "U8", "F16", "BF16", "f32_to_bf16_bits",
           "bf16_bits_to_f32"]
