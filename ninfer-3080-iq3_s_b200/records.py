"""The compact tile record at every code width (2, 3, 4, 5, 6, 8 bits) on the GPU: kvb_records_encode / _decode.

A record is  payload (LSB-first bit string, 16 * bits bytes per row) || scale_axis[128] || zp_axis[128] ||
other_axis[128]  (fp16 axes) for one 128 x 128 fp32 matrix; the reference's host oracle writes the same bytes
(kvarn-evidence/oracle/bee_oracle.cpp:152-172, 309-374).  No variance balancing here (other_axis = 1).
"""
import ctypes as C

import torch

from . import capi


def record_bytes(bits: int) -> int:
    n = capi.load().kvb_record_bytes(bits)
    if n == 0:
        raise ValueError(f"{bits}-bit codes: the record exists for 2, 3, 4, 5, 6 and 8 bits")
    return n


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def encode(tiles: torch.Tensor, bits: int) -> torch.Tensor:
    """tiles: [n, 128, 128] fp32 on the device -> uint8 [n, record_bytes(bits)]."""
    if tiles.dtype != torch.float32 or tiles.dim() != 3 or tuple(tiles.shape[1:]) != (128, 128) or not tiles.is_cuda:
        raise ValueError("tiles: a CUDA float32 tensor [n, 128, 128]")
    tiles = tiles.contiguous()
    out = torch.empty((tiles.shape[0], record_bytes(bits)), dtype=torch.uint8, device=tiles.device)
    capi.check(capi.load().kvb_records_encode(C.c_void_p(tiles.data_ptr()), tiles.shape[0], bits, C.c_void_p(out.data_ptr()), _stream()))
    return out


def decode(records: torch.Tensor, bits: int) -> torch.Tensor:
    """records: uint8 [n, record_bytes(bits)] on the device -> fp32 [n, 128, 128]."""
    if records.dtype != torch.uint8 or records.dim() != 2 or records.shape[1] != record_bytes(bits) or not records.is_cuda:
        raise ValueError(f"records: a CUDA uint8 tensor [n, {record_bytes(bits)}]")
    records = records.contiguous()
    out = torch.empty((records.shape[0], 128, 128), dtype=torch.float32, device=records.device)
    capi.check(capi.load().kvb_records_decode(C.c_void_p(records.data_ptr()), records.shape[0], bits, C.c_void_p(out.data_ptr()), _stream()))
    return out
