"""bf16 <-> float32 on numpy arrays (bf16 travels as uint16 bit patterns; round to nearest even)."""
import numpy as np


def to_bf16(x) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def from_bf16(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
