"""Independent numpy restatement of the three block decoders, written from the format
definitions rather than from the oracle's C, as a second opinion in the oracle's own tests."""
import numpy as np


def _f16(lo, hi):
    return (lo.astype(np.uint16) | (hi.astype(np.uint16) << 8)).view(np.float16).astype(np.float32)


def dequant_q8_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 34)
    d = _f16(b[:, 0], b[:, 1])
    q = b[:, 2:].view(np.int8).astype(np.float32)
    return (q * d[:, None]).astype(np.float32).ravel()


def dequant_q4_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 18)
    d = _f16(b[:, 0], b[:, 1])
    qs = b[:, 2:]
    lo = (qs & 0x0F).astype(np.int32) - 8
    hi = (qs >> 4).astype(np.int32) - 8
    q = np.concatenate([lo, hi], axis=1).astype(np.float32)
    return (q * d[:, None]).astype(np.float32).ravel()


def dequant_q4_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 144)
    d = _f16(b[:, 0], b[:, 1])
    dmin = _f16(b[:, 2], b[:, 3])
    s = b[:, 4:16].astype(np.int32)
    qs = b[:, 16:]
    sc = np.empty((b.shape[0], 8), dtype=np.int32)
    mn = np.empty((b.shape[0], 8), dtype=np.int32)
    for j in range(8):
        if j < 4:
            sc[:, j] = s[:, j] & 63
            mn[:, j] = s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    out = np.empty((b.shape[0], 256), dtype=np.float32)
    for j in range(8):
        chunk = qs[:, (j // 2) * 32:(j // 2) * 32 + 32]
        q = (chunk & 0xF) if j % 2 == 0 else (chunk >> 4)
        t = (d * sc[:, j].astype(np.float32)).astype(np.float32)
        t = (t[:, None] * q.astype(np.float32)).astype(np.float32)
        u = (dmin * mn[:, j].astype(np.float32)).astype(np.float32)
        out[:, j * 32:(j + 1) * 32] = (t - u[:, None]).astype(np.float32)
    return out.ravel()


DEQUANT = {8: dequant_q8_0, 2: dequant_q4_0, 12: dequant_q4_k}
