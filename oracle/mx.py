"""MXFP8-E4M3 / MXFP4-E2M1 block quantization with E8M0 scales, on CPU.

TEST INFRASTRUCTURE.  PARITY UNPINNED: the reference contains no MX code
(amct_pytorch/utils/vars.py:19-20 admits only int8/int4).  This restates the
public OCP Microscaling (MX) v1.0 conversion rule for a block of 32 values
along K:

    shared_exp = floor(log2(max|v|)) - emax_elem      (emax: 8 for E4M3, 2 for E2M1)
    scale byte = clamp(shared_exp, -127, 127) + 127   (E8M0, value 2^(byte-127))
    element    = saturating round-to-nearest-even of v * 2^-shared_exp

Build decisions where the rule is silent: an all-zero block gets scale byte 0;
a block holding NaN or Inf gets scale byte 0xFF and elements 0x7F (E4M3 NaN) /
saturated values (E2M1 has no NaN).  FP4 codes are packed two per byte, even
K index in the low nibble.
"""
import numpy as np
import torch

BLOCK = 32
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def _shared_exp(amax, emax_elem):
    """floor(log2(amax)) - emax_elem, clamped; amax == 0 -> -127."""
    _, e = np.frexp(amax.astype(np.float32))            # amax = m * 2^e, m in [0.5, 1)
    se = e.astype(np.int32) - 1 - emax_elem
    se = np.where(amax == 0, -127, se)
    return np.clip(se, -127, 127)


def _e2m1_codes(v):
    """RNE onto the E2M1 grid with saturation; returns 4-bit codes (sign in bit 3)."""
    a = np.minimum(np.abs(v), 6.0).astype(np.float32)
    idx = np.searchsorted(E2M1_GRID, a, side='left')          # first grid >= a
    idx = np.clip(idx, 1, 7)
    lo, hi = E2M1_GRID[idx - 1], E2M1_GRID[idx]
    dlo, dhi = a - lo, hi - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (idx % 2 == 0))   # tie -> even code
    code = np.where(pick_hi, idx, idx - 1).astype(np.uint8)
    return code | (np.signbit(v).astype(np.uint8) << 3)


def quantize(x, fmt):
    """x: torch [R, K] (K % 32 == 0) -> (payload uint8, scales uint8 [R, K/32]).

    fmt 'fp8': payload [R, K] E4M3 bit patterns.  fmt 'fp4': payload [R, K/2].
    """
    r, k = x.shape
    v = x.float().numpy().reshape(r, k // BLOCK, BLOCK)
    bad = ~np.isfinite(v).all(axis=-1)
    amax = np.abs(np.where(np.isfinite(v), v, 0)).max(axis=-1)
    emax = 8 if fmt == 'fp8' else 2
    se = _shared_exp(amax, emax)
    scales = (se + 127).astype(np.uint8)
    scales[bad] = 0xFF
    scaled = v * np.ldexp(np.float32(1), -se)[..., None].astype(np.float32)
    if fmt == 'fp8':
        t = torch.from_numpy(np.clip(scaled, -448.0, 448.0).astype(np.float32))
        q = t.to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
        q[bad] = 0x7F
        payload = q.reshape(r, k)
    else:
        c = _e2m1_codes(np.where(np.isnan(scaled), 0, scaled)).reshape(r, k)
        payload = c[:, 0::2] | (c[:, 1::2] << 4)
    return torch.from_numpy(payload), torch.from_numpy(scales)


def dequantize(payload, scales, fmt):
    """Exact fp32 values of an MX tensor."""
    sc = np.ldexp(np.float32(1), scales.numpy().astype(np.int32) - 127).astype(np.float32)
    if fmt == 'fp8':
        el = payload.view(torch.float8_e4m3fn).float().numpy()
    else:
        p = payload.numpy()
        c = np.stack((p & 0xF, p >> 4), axis=-1).reshape(p.shape[0], -1)
        el = E2M1_GRID[c & 7] * np.where(c & 8, -1.0, 1.0).astype(np.float32)
    r, k = el.shape
    out = el.reshape(r, k // BLOCK, BLOCK) * sc[..., None]
    return torch.from_numpy(out.reshape(r, k).astype(np.float32))


def gemm(a_payload, a_scales, b_payload, b_scales, fmt):
    """Block-scaled GEMM reference: y[m, n] = sum_k a[m, k] * b[n, k], fp64 accumulation
    of exactly dequantized operands (the tensor-core result is compared within a
    floating-point tolerance; accumulation order is not part of the contract)."""
    a = dequantize(a_payload, a_scales, fmt).double()
    b = dequantize(b_payload, b_scales, fmt).double()
    return (a @ b.t()).float()
