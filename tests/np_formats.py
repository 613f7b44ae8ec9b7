"""Independent numpy restatement of the block decoders, written from the format
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


def _k4_scales_mins(s):
    """The 6-bit scales and minima of eight sub-blocks from 12 packed bytes (rows of s)."""
    sc = np.empty((s.shape[0], 8), dtype=np.int32)
    mn = np.empty((s.shape[0], 8), dtype=np.int32)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def dequant_q4_1(raw: np.ndarray) -> np.ndarray:
    """20 bytes per 32 elements: fp16 d, fp16 m, nibbles packed like Q4_0; (q * d) + m, q unsigned."""
    b = raw.reshape(-1, 20)
    d = _f16(b[:, 0], b[:, 1])
    m = _f16(b[:, 2], b[:, 3])
    qs = b[:, 4:]
    q = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32)
    t = (q * d[:, None]).astype(np.float32)
    return (t + m[:, None]).astype(np.float32).ravel()


def dequant_q5_k(raw: np.ndarray) -> np.ndarray:
    """176 bytes per 256: d, dmin, 12 bytes of packed scales / minima, 32 bytes of fifth bits (bit j of byte p is
    element 32 j + p), 128 bytes of nibbles (byte 32 c + p: low nibble element 64 c + p, high nibble 64 c + 32 + p)."""
    b = raw.reshape(-1, 176)
    d = _f16(b[:, 0], b[:, 1])
    dmin = _f16(b[:, 2], b[:, 3])
    sc, mn = _k4_scales_mins(b[:, 4:16].astype(np.int32))
    qh = b[:, 16:48].astype(np.int32)
    qs = b[:, 48:].astype(np.int32).reshape(-1, 4, 32)
    nib = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32)          # [block][sub-block][position]
    fifth = (qh[:, None, :] >> np.arange(8)[None, :, None]) & 1             # bit j of qh[p] belongs to sub-block j
    q = (nib + 16 * fifth).astype(np.float32)
    t = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    t = (t[:, :, None] * q).astype(np.float32)
    u = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    return (t - u[:, :, None]).astype(np.float32).reshape(-1)


def dequant_q6_k(raw: np.ndarray) -> np.ndarray:
    """210 bytes per 256: 128 bytes ql, 64 bytes qh, 16 signed scales, fp16 d. Per half of 128 elements: group g of 32
    takes nibble (g >> 1) of ql[64 h + 32 (g & 1) + p] and bits 2g, 2g+1 of qh[32 h + p]; value - 32; scale of every 16."""
    b = raw.reshape(-1, 210)
    nb = b.shape[0]
    ql = b[:, 0:128].astype(np.int32).reshape(nb, 2, 2, 32)                 # [half][g & 1][p]
    qh = b[:, 128:192].astype(np.int32).reshape(nb, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.float32)                     # one per 16 elements, in element order
    d = _f16(b[:, 208], b[:, 209])
    out = np.empty((nb, 2, 4, 32), dtype=np.int32)
    for g in range(4):
        low = (ql[:, :, g & 1, :] >> (4 * (g >> 1))) & 0xF
        out[:, :, g, :] = (low | (((qh >> (2 * g)) & 3) << 4)) - 32
    q = out.reshape(nb, 16, 16).astype(np.float32)
    t = (d[:, None] * sc).astype(np.float32)
    return (t[:, :, None] * q).astype(np.float32).reshape(-1)


DEQUANT = {8: dequant_q8_0, 2: dequant_q4_0, 12: dequant_q4_k, 3: dequant_q4_1, 13: dequant_q5_k, 14: dequant_q6_k}
