"""NumPy twin of the C oracle -- TEST INFRASTRUCTURE ONLY.

An independent float32 restatement of the reference's quantizers and dequantizers
(src/packed_tensor.rs, src/dtypes/*.rs of fastnn).  The reference pins no packed bytes or
scales for random weights, so the C oracle and this twin are written separately and must
agree bit for bit (tests/test_oracle_twin.py).  Vectorised where the order of f32
operations does not matter, sequential (np.cumsum) where it does.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
FP4_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)


def _round_half_away(x: np.ndarray) -> np.ndarray:
    # Rust f32::round.  trunc(x + copysign(0.5, x)) is wrong for 0.49999997; do it exactly.
    t = np.trunc(x)
    frac = np.abs(x - t)
    return np.where(frac >= F32(0.5), t + np.sign(x).astype(F32), t).astype(F32)


# ---------------------------------------------------------------- e4m3 / e2m1

def e4m3_decode_table() -> np.ndarray:
    """src/dtypes/f8x4.rs:23-38 evaluated for all 256 codes."""
    out = np.zeros(256, dtype=F32)
    for b in range(256):
        sign = F32(-1.0) if b & 0x80 else F32(1.0)
        e = (b >> 3) & 0xF
        m = F32(b & 7)
        if e == 0:
            out[b] = F32(0.0) * sign if m == 0 else sign * F32(2.0 ** -6) * (m / F32(8.0))
        elif e == 0xF:
            out[b] = np.nan
        else:
            out[b] = sign * F32(2.0 ** (e - 7)) * (F32(1.0) + m / F32(8.0))
    return out


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """src/dtypes/f8x4.rs:41-77, vectorised.  floor(log2(x)) is taken from the f32
    exponent bits (identical for normal inputs; inputs below 2^-6 use the subnormal arm)."""
    v = np.asarray(v, dtype=F32)
    out = np.zeros(v.shape, dtype=np.uint8)
    nan = np.isnan(v)
    sign = np.where(v < 0, 0x80, 0).astype(np.uint8)
    a = np.minimum(np.abs(v), F32(240.0)).astype(F32)
    zero = a == 0
    sub = (a < F32(0.015625)) & ~zero
    m_sub = np.clip(_round_half_away(a * F32(512.0)), 0, 255).astype(np.int64)
    sub_code = np.where(m_sub >= 8, 0x08, m_sub).astype(np.uint8)
    bits = a.view(np.uint32).astype(np.int64)
    e = ((bits >> 23) & 0xFF) - 127
    pow2 = np.ldexp(F32(1.0), e.astype(np.int32)).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        norm = (a / pow2).astype(F32)
    mant = np.clip(_round_half_away((norm - F32(1.0)) * F32(8.0)), 0, 255).astype(np.int64)
    biased = e + 7
    bump = mant >= 8
    nb = np.where(bump, biased + 1, biased)
    code = np.where(nb >= 15, 0x7B, (nb << 3) | np.where(bump, 0, mant)).astype(np.uint8)
    out = np.where(sub, sub_code, code).astype(np.uint8)
    out = np.where(zero, 0, out).astype(np.uint8) | sign
    out = np.where(zero, np.where(np.signbit(v), 0x80, 0), out).astype(np.uint8)
    out = np.where(nan, 0x7F, out).astype(np.uint8)
    return out


def fp4_decode_table() -> np.ndarray:
    """src/dtypes/f4x8.rs:25-39."""
    t = np.zeros(16, dtype=F32)
    for c in range(16):
        mag = FP4_MAG[c & 7]
        t[c] = -mag if (c & 8) and (c & 7) else mag
    return t


def fp4_encode(v: np.ndarray) -> np.ndarray:
    """src/dtypes/f4x8.rs:49-70: nearest magnitude, first minimum wins."""
    v = np.asarray(v, dtype=F32)
    a = np.abs(v)
    d = np.abs(a[..., None] - FP4_MAG[None, :]).astype(F32)
    best = np.argmin(d, axis=-1)  # first minimum
    neg = np.signbit(v) & (best != 0)
    code = (best | np.where(neg, 8, 0)).astype(np.uint8)
    return np.where(np.isnan(v), 0, code).astype(np.uint8)


# ---------------------------------------------------------------- word packing

def _pad_rows(vals: np.ndarray, items: int) -> np.ndarray:
    n, k = vals.shape
    kp = -(-k // items)
    out = np.zeros((n, kp * items), dtype=vals.dtype)
    out[:, :k] = vals
    return out.reshape(n, kp, items)


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """codes: [N, K] unsigned lane codes -> [N*kp + 16] u32 (lane i at bits [bits*i, ...))."""
    items = 32 // bits
    lanes = _pad_rows(codes.astype(np.uint32), items)
    shifts = (np.arange(items, dtype=np.uint32) * np.uint32(bits))[None, None, :]
    words = np.bitwise_or.reduce(lanes << shifts, axis=-1).astype(np.uint32)
    return np.concatenate([words.reshape(-1), np.zeros(16, dtype=np.uint32)])


def int_codes(lane_vals: np.ndarray, bits: int) -> np.ndarray:
    """src/dtypes/i4x8.rs:33-40 / i8x4.rs:33-41: clamp, round half away, two's complement."""
    lo, hi = (-8.0, 7.0) if bits == 4 else (-128.0, 127.0)
    q = _round_half_away(np.clip(lane_vals, F32(lo), F32(hi)))
    q = np.where(np.isnan(lane_vals), 0, q).astype(np.int64)
    return (q & ((1 << bits) - 1)).astype(np.uint32)


# ---------------------------------------------------------------- quantizers

def quantize_int_asym(w_nk: np.ndarray, bits: int):
    """src/packed_tensor.rs:852-1049, integer branch (:966-974)."""
    w = np.asarray(w_nk, dtype=F32)
    umax = F32((1 << bits) - 1)
    bias = F32(1 << (bits - 1))
    mn = w.min(axis=1).astype(F32)
    mx = w.max(axis=1).astype(F32)
    rng = (mx - mn).astype(F32)
    init = (rng / umax).astype(F32)
    lo = (mn - init).astype(F32)
    hi = (mx + init).astype(F32)
    scale = ((hi - lo).astype(F32) / umax).astype(F32)
    zero = (lo + (bias * scale).astype(F32)).astype(F32)
    flat = rng == 0
    scale = np.where(flat, F32(1.0), scale).astype(F32)
    zero = np.where(flat, F32(0.0), zero).astype(F32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale != 0, F32(1.0) / scale, F32(0.0)).astype(F32)
    lane = ((w - zero[:, None]).astype(F32) * inv[:, None]).astype(F32)
    return pack_codes(int_codes(lane, bits), bits), scale, zero


def quantize_fp4_asym(w_nk: np.ndarray):
    """src/packed_tensor.rs:950-965: zero = sequential-sum mean, scale = maxdev / 4."""
    w = np.asarray(w_nk, dtype=F32)
    n, k = w.shape
    mn = w.min(axis=1).astype(F32)
    mx = w.max(axis=1).astype(F32)
    rng = (mx - mn).astype(F32)
    seq_sum = np.cumsum(w, axis=1, dtype=F32)[:, -1]  # cumsum adds strictly left to right
    mean = (seq_sum / F32(k)).astype(F32)
    dev = np.maximum(np.abs(mean - mn), np.abs(mx - mean)).astype(F32)
    max_dev = np.where(dev == 0, F32(1e-10), dev).astype(F32)
    scale = (max_dev / F32(4.0)).astype(F32)
    zero = mean
    flat = rng == 0
    scale = np.where(flat, F32(1.0), scale).astype(F32)
    zero = np.where(flat, F32(0.0), zero).astype(F32)
    inv = np.where(scale != 0, F32(1.0) / scale, F32(0.0)).astype(F32)
    lane = ((w - zero[:, None]).astype(F32) * inv[:, None]).astype(F32)
    return pack_codes(fp4_encode(lane), 4), scale, zero


def quantize_f8_sym(w_nk: np.ndarray):
    """src/packed_tensor.rs:661-742."""
    w = np.asarray(w_nk, dtype=F32)
    max_abs = np.abs(w).max(axis=1).astype(F32)
    scale = np.where(max_abs == 0, F32(1.0), max_abs / F32(240.0)).astype(F32)
    inv = np.where(scale != 1, F32(1.0) / scale, F32(1.0)).astype(F32)
    lane = (w * inv[:, None]).astype(F32)
    return pack_codes(e4m3_encode(lane), 8), scale


def kmeans16(values: np.ndarray, iters: int = 30) -> np.ndarray:
    """src/packed_tensor.rs:18-75."""
    v = np.asarray(values, dtype=F32).reshape(-1)
    n = v.size
    c = np.zeros(16, dtype=F32)
    if n == 0:
        return c
    if n == 1:
        return np.full(16, v[0], dtype=F32)
    s = np.sort(v, kind="stable")
    for i in range(16):
        pct = (F32(i) + F32(0.5)) / F32(16.0)
        idx = int(F32(pct) * F32(n))
        c[i] = s[min(idx, n - 1)]
    for _ in range(iters):
        d = np.abs(v[:, None] - c[None, :]).astype(F32)
        a = np.argmin(d, axis=1)  # first minimum
        for ci in range(16):
            sel = v[a == ci]
            if sel.size:
                c[ci] = np.cumsum(sel, dtype=F32)[-1] / F32(sel.size)
    return np.sort(c)


def quantize_codebook(w_nk: np.ndarray, qblock: int = 32):
    """src/packed_tensor.rs:1209-1313."""
    w = np.asarray(w_nk, dtype=F32)
    n, k = w.shape
    bpr = -(-k // qblock)
    pad = np.zeros((n, bpr * qblock), dtype=F32)
    pad[:, :k] = w
    blocks = pad.reshape(n, bpr, qblock)
    bs = np.abs(blocks).max(axis=2).astype(F32)  # padding zeros never raise a max
    with np.errstate(divide="ignore"):
        inv = np.where(bs > 0, F32(1.0) / bs, F32(0.0)).astype(F32)
    normalized = (blocks * inv[:, :, None]).astype(F32).reshape(n, bpr * qblock)[:, :k]
    cb = kmeans16(normalized.reshape(-1))
    d = np.abs(normalized[:, :, None] - cb[None, None, :]).astype(F32)
    idx = np.argmin(d, axis=2).astype(np.uint32)
    return pack_codes(idx, 4), bs.reshape(-1), cb


def unpack_codes(words: np.ndarray, n: int, k: int, bits: int) -> np.ndarray:
    items = 32 // bits
    kp = -(-k // items)
    w = np.asarray(words[: n * kp], dtype=np.uint32).reshape(n, kp, 1)
    shifts = (np.arange(items, dtype=np.uint32) * np.uint32(bits))[None, None, :]
    codes = (w >> shifts) & np.uint32((1 << bits) - 1)
    return codes.reshape(n, kp * items)[:, :k]


def dequant(fmt: str, words, n, k, scales, zeros=None, codebook=None, qblock=32) -> np.ndarray:
    """src/packed_tensor.rs:469-521: unpack(q) * scale + zero as two f32 roundings."""
    if fmt == "i4cb":
        idx = unpack_codes(words, n, k, 4)
        blk = (np.arange(k) // qblock)[None, :]
        bs = np.asarray(scales, dtype=F32).reshape(n, -1)
        return (np.take_along_axis(bs, np.broadcast_to(blk, (n, k)), axis=1)
                * np.asarray(codebook, dtype=F32)[idx]).astype(F32)
    if fmt == "i8":
        u = unpack_codes(words, n, k, 8).astype(np.int64)
        vals = np.where(u >= 128, u - 256, u).astype(F32)
    elif fmt == "i4":
        u = unpack_codes(words, n, k, 4).astype(np.int64)
        vals = np.where(u >= 8, u - 16, u).astype(F32)
    elif fmt == "f8":
        vals = e4m3_decode_table()[unpack_codes(words, n, k, 8)]
    elif fmt == "f4":
        vals = fp4_decode_table()[unpack_codes(words, n, k, 4)]
    else:
        raise ValueError(fmt)
    s = np.asarray(scales, dtype=F32)[:, None]
    z = (np.zeros(n, dtype=F32) if zeros is None or len(zeros) == 0
         else np.asarray(zeros, dtype=F32))[:, None]
    return ((vals * s).astype(F32) + z).astype(F32)
