"""Seeded synthetic inputs shaped like the configurations the benchmark names, plus small helpers."""
import numpy as np

BASE_SEED = 20251125


def rng(idx):
    return np.random.default_rng(BASE_SEED + idx)


def rescale_params(r, channels):
    """Per-channel RESCALE operands: multiplier U[2^30, 2^31-1], shift U[30, 40]."""
    mult = r.integers(1 << 30, (1 << 31) - 1, size=channels, endpoint=True, dtype=np.int64).astype(np.int32)
    shift = r.integers(30, 40, size=channels, endpoint=True, dtype=np.int64).astype(np.int8)
    return mult, shift


def conv_int8_case(r, N, IH, IW, IC, OC, KH, KW, bias_range=32768):
    x = r.integers(-128, 127, size=(N, IH, IW, IC), endpoint=True, dtype=np.int64).astype(np.int8)
    w = r.integers(-127, 127, size=(OC, KH, KW, IC), endpoint=True, dtype=np.int64).astype(np.int8)
    b = r.integers(-bias_range, bias_range - 1, size=OC, endpoint=True, dtype=np.int64).astype(np.int32)
    return x, w, b


def to_bf16_bits(a):
    """float32 array -> bfloat16 bit patterns (round to nearest even), as uint16."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    u = (u + 0x7FFF + lsb) >> 16
    return u.astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)
