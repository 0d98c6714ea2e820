"""Helpers shared by the GPU parity tests: seeded inputs, torch <-> numpy views, oracle access."""
import numpy as np
import torch

from oracle import nvfp4_oracle as O


def to_dev(x_f32):
    """float32 numpy (bf16-representable values) -> bf16 CUDA tensor, bit-exact."""
    bits = O.f32_to_bf16_bits(np.asarray(x_f32, dtype=np.float32))
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def bf16_round(x_f32):
    """Round a float32 numpy array to bf16-representable float32 values."""
    return O.bf16_bits_to_f32(O.f32_to_bf16_bits(np.asarray(x_f32, dtype=np.float32)))


def u8(t):
    return t.view(torch.uint8).cpu().numpy()


def student_t(rng, shape, df=3):
    return (rng.standard_normal(shape) / np.sqrt(rng.chisquare(df, shape) / df)).astype(np.float32)


def make_x(seed, R, C, outliers=8):
    """BASELINE config-1 style activations: N(0,1), a few columns x30."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((R, C)).astype(np.float32)
    if outliers:
        x[:, rng.permutation(C)[:outliers]] *= 30
    return bf16_round(x)


def make_w(seed, N, K, std=0.02):
    rng = np.random.default_rng(seed)
    return bf16_round(rng.standard_normal((N, K)).astype(np.float32) * std)


def make_dy(seed, T, N):
    rng = np.random.default_rng(seed)
    return bf16_round(student_t(rng, (T, N)) * 1e-3)


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))
