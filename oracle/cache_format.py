"""The decode cache format on the CPU, in numpy. Test infrastructure only.

Every function follows the reference's torch quantisers one rounded fp32
operation at a time, so its outputs are the reference's bits:
`src/fold_attention/decode/cache.py` and `src/fold_attention/utils.py`.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32
FMAX = F32(448.0)
# cache.py:29  `1/127` rounded once to fp32
INV127 = F32(1.0) / F32(127.0)
KBR = F32(256.0)
LOG2E = 1.4426950408889634
# decode/write.py:730  a prompt's reductions run over chunks of this many tokens
CHUNK = 256
NT = 128


def hadamard(x: np.ndarray) -> np.ndarray:
    """Orthonormal Sylvester-Hadamard over the last axis as a fixed-order
    butterfly in fp32 (utils.py:60-78): stage h pairs element i with i+h."""
    d = x.shape[-1]
    if d & (d - 1):
        raise ValueError(f"a Sylvester Hadamard needs a power of two, got {d}")
    y = np.ascontiguousarray(x, dtype=F32).reshape(-1, d)
    h = 1
    while h < d:
        y = y.reshape(-1, d // (2 * h), 2, h)
        a, b = y[:, :, 0], y[:, :, 1]
        y = np.stack((a + b, a - b), 2).astype(F32)
        h *= 2
    return (y.reshape(x.shape) * F32(1.0 / math.sqrt(d))).astype(F32)


def swizzle_of(row_bytes: int):
    """(units, shift, atom bytes) of a row's XOR swizzle (cache.py:36-50)."""
    nu = min(row_bytes // 16, 8)
    if nu < 1 or nu & (nu - 1):
        raise ValueError(f"a {row_bytes}-byte row has no power-of-two unit count")
    return nu, 3 - (nu.bit_length() - 1), nu * 128


def swizzle_units(plane: np.ndarray, slot: np.ndarray) -> np.ndarray:
    """`plane` (N, D) bytes with 16-byte unit u of row r moved to
    `u ^ ((slot[r] >> shift) & (units-1))` (cache.py:53-69, 389-396)."""
    n, d = plane.shape
    nu, sh, _ = swizzle_of(d)
    v = plane.reshape(n, nu, 16)
    idx = np.arange(nu)[None, :] ^ ((slot.astype(np.int64) >> sh) & (nu - 1))[:, None]
    # stored[u] = source[u ^ x]  (a gather; XOR is an involution so the two
    # readings of the rule coincide)
    return np.take_along_axis(v, idx[:, :, None], 1).reshape(n, d)


def key_scale(amax: np.ndarray) -> np.ndarray:
    """`amax/127` as one fp32 multiply, rounded UP to the next bf16
    (cache.py:97-106). Returned as fp32 whose low 16 bits are zero."""
    e = (np.maximum(amax.astype(F32), F32(1e-30)) * INV127).astype(F32)
    b = e.view(np.int32)
    return ((b + 0xFFFF) & np.int32(-65536)).view(F32)


def int8_planes(x: np.ndarray, e: np.ndarray):
    """x = e (a + b/256): one rounded reciprocal and a multiply per plane
    (cache.py:72-78)."""
    x = x.astype(F32)
    e = e.astype(F32)
    pa = np.clip(np.rint((x * (F32(1.0) / e)).astype(F32)), -128, 127).astype(F32)
    r = (x - (pa * e).astype(F32)).astype(F32)
    pb = np.clip(np.rint((r * (KBR / e)).astype(F32)), -128, 127)
    return pa.astype(np.int8), pb.astype(np.int8)


def key_planes(k: np.ndarray, rot: bool = True):
    """Keys' two int8 planes (unswizzled) and each key's scale (cache.py:109-119)."""
    x = hadamard(k) if rot else k.astype(F32)
    e = key_scale(np.abs(x).max(-1, keepdims=True))
    pa, pb = int8_planes(x, e)
    return pa, pb, e[..., 0]


def quantize_q(q: np.ndarray, head_dim: int | None = None, rot: bool = True):
    """Query rows -> (plane A, plane B, fp32 scale). `q` is the raw query; it
    is first scaled by fp32(LOG2E/sqrt(D)) (decode/quant.py:130-139), rotated,
    and scaled by amax * fp32(1/127) (a multiply, as the device and CUDA torch
    do it; cache.py:92 read on a CPU would divide)."""
    d = q.shape[-1] if head_dim is None else head_dim
    x = (q.astype(F32) * F32(LOG2E / math.sqrt(d))).astype(F32)
    return quantize_kq(x, rot)


def quantize_kq(x: np.ndarray, rot: bool = True):
    """cache.py:88-94 on an already scaled query."""
    if rot:
        x = hadamard(x)
    e = (np.maximum(np.abs(x).max(-1, keepdims=True), F32(1e-30)) * INV127).astype(F32)
    pa, pb = int8_planes(x, e)
    return pa, pb, e[..., 0]


# ---------------------------------------------------------------- E4M3 ----

def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float64)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        ex, m = (b >> 3) & 0xF, b & 7
        if ex == 0:
            v = m / 8.0 * 2.0**-6
        elif ex == 15 and m == 7:
            v = float("nan")
        else:
            v = (1 + m / 8.0) * 2.0 ** (ex - 7)
        t[b] = s * v
    return t.astype(F32)


E4M3_VALUES = _e4m3_table()


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 (already clamped to +-448) -> e4m3fn bits, round to nearest even,
    the sign kept on zeros: torch's `.to(float8_e4m3fn)` and
    `cvt.rn.satfinite.e4m3x2.f32` agree on this range."""
    x = x.astype(F32)
    sign = np.signbit(x).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    _, ex = np.frexp(a)
    e = np.maximum(ex - 1, -6)
    q = np.ldexp(1.0, e - 3)
    v = np.rint(a / q) * q  # exact: q is a power of two
    _, ex2 = np.frexp(v)
    e2 = ex2 - 1
    den = e2 < -6
    bits_den = np.rint(v * 2.0**9).astype(np.int64)
    safe = np.where(v > 0, v, 1.0)
    man = np.rint((safe / np.ldexp(1.0, np.where(v > 0, e2, 0)) - 1.0) * 8).astype(np.int64)
    bits_nrm = ((np.where(v > 0, e2, -7) + 7) << 3) | man
    bits = np.where(v == 0, 0, np.where(den, bits_den, bits_nrm))
    return (bits.astype(np.uint8) | sign).astype(np.uint8)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[b.astype(np.uint8)]


def e4m3_planes(v: np.ndarray, e: float):
    """V's two e4m3 planes under the power-of-two scale e (cache.py:81-85)."""
    s = (v.astype(F32) / F32(e)).astype(F32)
    pa = e4m3_encode(np.clip(s, -FMAX, FMAX))
    r = (s - e4m3_decode(pa)).astype(F32)
    pb = e4m3_encode(np.clip((r * F32(8.0)).astype(F32), -FMAX, FMAX))
    return pa, pb


def pow2_ceil(x: np.ndarray) -> np.ndarray:
    """Least power of two >= a positive normal x, from its bits (decode/ptx.py:513-524)."""
    b = np.asarray(x, dtype=F32).view(np.uint32)
    e = b & np.uint32(0x7F800000)
    e = np.where(b & np.uint32(0x7FFFFF), e + np.uint32(0x800000), e).astype(np.uint32)
    return e.view(F32)


def v_scale_rule(vmax: float, headroom: float) -> np.float32:
    """The layer's V scale from the prompts' largest |v| (decode/write.py:818-822)."""
    t = (F32(vmax) * F32(headroom)).astype(F32)
    t = (t * F32(1.0 / 448.0)).astype(F32)
    return pow2_ceil(np.maximum(t, F32(1e-30)))[()]


# ------------------------------------------------------------ page rows ----

def page_row(page_table: np.ndarray, b, h, pos, page_size: int, n_kv_heads: int):
    """Pool row of request b, KV head h, position pos, and its slot in the
    page (decode/device.py:110-114, write.py:141-151)."""
    pg = page_table[b, pos // page_size].astype(np.int64)
    off = pos % page_size
    return (pg * n_kv_heads + h) * page_size + off, off


def write_rows(pool: dict, k, v, ev, row, off, rot=True):
    """Quantise (N, H, D) keys and values into pool rows `row` (N, H); `off`
    (N,) is each token's page slot (cache.py:370-396). `pool` holds ka, kb
    (int8), ek (fp32 view of bf16 scales), va, vb (uint8 e4m3 bits or None for
    a 16-bit V, in which case va takes `v` itself as fp32)."""
    n, h, d = k.shape
    pa, pb, e = key_planes(k, rot)
    r = row.reshape(-1)
    slot = np.repeat(off, h)
    pool["ek"][r] = e.reshape(-1)
    pool["ka"][r] = swizzle_units(pa.reshape(n * h, d).view(np.uint8), slot).view(np.int8)
    pool["kb"][r] = swizzle_units(pb.reshape(n * h, d).view(np.uint8), slot).view(np.int8)
    if pool.get("vb") is None:
        pool["va"][r] = v.reshape(n * h, d)
    else:
        qa, qb = e4m3_planes(v, ev)
        pool["va"][r] = qa.reshape(n * h, d)
        pool["vb"][r] = qb.reshape(n * h, d)


def append_vsum(vsum, v_new, pos, ev):
    """The append's running V sum and mean (decode/write.py:141-151):
    vsum += v; vmean = vsum / (float(pos+1) * ev)."""
    s = (vsum.astype(F32) + v_new.astype(F32)).astype(F32)
    n = (np.asarray(pos + 1, dtype=F32) * F32(ev)).astype(F32)
    return s, (s / n).astype(F32)


def prompt_vsum(v: np.ndarray, lens, ev: float):
    """A prompt's per-(request, head) V sum and mean in the reference's fixed
    order (decode/write.py:733-845): 256-token chunks from the request's start;
    inside a chunk, slot j of R = 128/(D/16) adds rows j, j+R, j+2R, ... in
    turn, the slots are then added j = 0..R-1, and the chunks in order."""
    total, hkv, d = v.shape
    rpb = NT // (d // 16)
    out_s = np.zeros((len(lens), hkv, d), F32)
    out_m = np.zeros_like(out_s)
    t0 = 0
    for b, n in enumerate(lens):
        acc = np.zeros((hkv, d), F32)
        for p0 in range(0, n, CHUNK):
            cnt = min(CHUNK, n - p0)
            x = v[t0 + p0 : t0 + p0 + cnt].astype(F32)
            part = np.zeros((rpb, hkv, d), F32)
            for it in range(CHUNK // rpb):
                lo = it * rpb
                if lo >= cnt:
                    break
                rows = x[lo : min(lo + rpb, cnt)]
                part[: rows.shape[0]] = (part[: rows.shape[0]] + rows).astype(F32)
            c = np.zeros((hkv, d), F32)
            for j in range(rpb):
                c = (c + part[j]).astype(F32)
            acc = (acc + c).astype(F32)
        out_s[b] = acc
        out_m[b] = (acc / (F32(n) * F32(ev)).astype(F32)).astype(F32)
        t0 += n
    return out_s.reshape(-1, d), out_m.reshape(-1, d)


def write_prompt(pool, k, v, lens, page_table, page_size, v8, v_headroom=2.0, v_scale=None):
    """decode/write.py:931-1009 on the CPU: returns the V scale; fills the pool
    planes, scales, vsum and vmean."""
    total, hkv, d = k.shape
    if v8:
        ev = float(v_scale) if v_scale is not None else float(
            v_scale_rule(float(np.abs(v.astype(F32)).max()), v_headroom))
    else:
        ev = 1.0
    req = np.repeat(np.arange(len(lens)), lens)
    cu = np.concatenate([[0], np.cumsum(lens)])
    pos = np.arange(total) - cu[req]
    row, off = page_row(page_table, req[:, None], np.arange(hkv)[None, :], pos[:, None],
                        page_size, hkv)
    write_rows(pool, k, v, ev, row, pos % page_size)
    pool["vsum"][: len(lens) * hkv], pool["vmean"][: len(lens) * hkv] = prompt_vsum(v, lens, ev)
    return ev
