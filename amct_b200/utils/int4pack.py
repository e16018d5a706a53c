"""The two packed forms of INT4 weight codes and the conversions between them (one-off layout work at convert / load
time, written with torch ops on whatever device holds the tensor).

``int4pack``  what ``torch_npu.npu_convert_weight_to_int4pack`` returns for the [K, N] int32 codes the reference hands it
              (amct_pytorch/deploy_op/weight_npu_quant_module.py:53-57) and what a deployed state dict therefore holds
              under ``quantized_weight``: int32 [K, N / 8], eight two's-complement nibbles per word along N, column
              8 j + i in bits [4 i, 4 i + 4) of word j.  (The reference's test double returns its input unchanged: int32
              [K, N]; ``codes_from_buffer`` accepts that form as well.)
``payload``   what this package's kernels read: uint8 [N, K / 2], two codes per byte along K, code + 8 (so that
              zero-points live in [0, 15]), even k in the low nibble.
"""
import torch


def to_int4pack(codes_kn):
    """[K, N] integer codes in [-8, 7] -> int32 [K, N / 8]."""
    k, n = codes_kn.shape
    if n % 8:
        raise ValueError(f'int4pack packs eight output channels per word: N = {n} is not a multiple of 8')
    nib = (codes_kn.to(torch.int64) & 0xF).reshape(k, n // 8, 8)
    shifts = torch.arange(0, 32, 4, device=codes_kn.device, dtype=torch.int64)
    word = (nib << shifts).sum(dim=-1)                                   # in [0, 2^32)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)           # the same 32 bits as a signed number
    return word.to(torch.int32)


def from_int4pack(packed_kn8):
    """int32 [K, N / 8] -> int8 codes [K, N] in [-8, 7]."""
    k, n8 = packed_kn8.shape
    shifts = torch.arange(0, 32, 4, device=packed_kn8.device, dtype=torch.int64)
    nib = (packed_kn8.to(torch.int64).unsqueeze(-1) >> shifts) & 0xF
    codes = torch.where(nib >= 8, nib - 16, nib)
    return codes.reshape(k, n8 * 8).to(torch.int8)


def to_payload(codes_nk):
    """[N, K] integer codes in [-8, 7] -> uint8 [N, K / 2] (code + 8, even k in the low nibble)."""
    n, k = codes_nk.shape
    if k % 2:
        raise ValueError(f'two codes per byte along K: K = {k} is odd')
    u = (codes_nk.to(torch.int16) + 8).to(torch.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).contiguous()


def from_payload(payload_nk2):
    """uint8 [N, K / 2] -> int8 codes [N, K]."""
    lo = (payload_nk2 & 0xF).to(torch.int8) - 8
    hi = (payload_nk2 >> 4).to(torch.int8) - 8
    return torch.stack((lo, hi), dim=-1).reshape(payload_nk2.shape[0], -1)


def codes_from_buffer(quantized_weight, n):
    """The [K, N] codes behind any form a ``quantized_weight`` buffer of an INT4 Linear with N output channels can have:
    int32 [K, N / 8] (int4pack), int32 or int8 [K, N] (unpacked, what the reference's test double leaves), or uint8
    [K / 2, N] (this package's payload viewed with the reference's axis order, as earlier versions stored it)."""
    q = quantized_weight
    if q.dtype == torch.uint8 and q.shape[1] == n:
        return from_payload(q.t().contiguous()).t()
    if q.dtype == torch.int32 and n % 8 == 0 and q.shape[1] == n // 8 and n // 8 != n:
        return from_int4pack(q)
    if q.shape[1] == n:
        return q.to(torch.int8)
    raise RuntimeError(f'quantized_weight of shape {tuple(q.shape)} and dtype {q.dtype} is not an INT4 weight with {n} output channels')
