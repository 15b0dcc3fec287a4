"""Shared helpers of the GPU parity tests: a device layer and its CPU-oracle twin on the same inputs."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402
from oracle import kvarn_oracle as orc  # noqa: E402

# Tolerance of the attention outputs against the oracle (fp32/double attention on the de-quantised cache):
# max-abs error <= 2^-10 of the largest reference magnitude, relative L2 <= 1e-3.
ATTN_MAX_ABS = 2.0 ** -10
ATTN_REL_L2 = 1e-3


def pkg():
    return entry.load_package()


def torch_dtype(dtype):
    import torch

    return torch.bfloat16 if dtype == 1 else torch.float16


def to_bits(x16: np.ndarray, dtype: int) -> np.ndarray:
    """fp16 values -> the 16-bit patterns fed to both sides (fp16, or bf16 by truncating fp32)."""
    if dtype == 0:
        return x16.view(np.uint16)
    return (x16.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)


def from_bits(bits: np.ndarray, dtype: int):
    import torch

    t = torch.from_numpy(bits.view(np.int16).copy())
    return t.view(torch.bfloat16 if dtype == 1 else torch.float16)


class Twin:
    """A CUDA layer and a CPU-oracle layer that receive identical appends."""

    def __init__(self, D=128, H=4, QH=24, capacity_tokens=4096, seed=0, dtype=0, iters=0, extra_pages=3):
        import torch

        lp = (capacity_tokens + 63) // 64 + 2
        lp += lp & 1
        self.D, self.H, self.QH, self.dtype = D, H, QH, dtype
        self.table = orc.shuffled_table(seed, lp, lp + extra_pages)
        self.cpu = orc.CpuLayer(D, H, lp + extra_pages, self.table, iters)
        self.dev = torch.device("cuda:0")
        self.gpu = pkg().KvarnLayer(D, H, QH, lp + extra_pages, torch.from_numpy(self.table), dtype=torch_dtype(dtype),
                                    sinkhorn_iters=iters, device="cuda:0")
        self.len = 0

    def append(self, k16: np.ndarray, v16: np.ndarray, pos0=None):
        import torch

        pos0 = self.len if pos0 is None else pos0
        kb, vb = to_bits(k16, self.dtype), to_bits(v16, self.dtype)
        self.cpu.append(kb, vb, pos0, self.dtype)
        n = kb.shape[0]
        self.gpu.append(from_bits(kb, self.dtype).to(self.dev), from_bits(vb, self.dtype).to(self.dev),
                        torch.arange(pos0, pos0 + n, dtype=torch.int32, device=self.dev))
        self.len = pos0 + n

    def planes_equal(self):
        g = self.gpu
        out = {}
        out["k_code"] = np.array_equal(g.k_code.cpu().numpy(), self.cpu.k_code)
        out["v_code"] = np.array_equal(g.v_code.cpu().numpy(), self.cpu.v_code)
        out["k_scale"] = np.array_equal(g.k_scale.cpu().numpy().view(np.uint16), self.cpu.k_scale)
        out["v_scale"] = np.array_equal(g.v_scale.cpu().numpy().view(np.uint16), self.cpu.v_scale)
        return out

    def stage_np(self):
        return self.gpu.stage.cpu().numpy().view(np.uint16).reshape(2, 2, self.H, 128, self.D)

    def live_stage_equal(self):
        live = self.len % 128
        slot = (self.len // 128) & 1
        return np.array_equal(self.stage_np()[:, slot, :, :live], self.cpu.stage[:, slot, :, :live])


# The prefill kernel rounds the de-quantised K and V tiles to fp16 before the tensor-core contraction (the decode
# kernel keeps them exact and splits q instead): max-abs <= 2^-8 of the largest reference magnitude, rel-L2 <= 5e-3.
PREFILL_MAX_ABS = 2.0 ** -8
PREFILL_REL_L2 = 5e-3


def attn_close(got: np.ndarray, want: np.ndarray, max_abs=ATTN_MAX_ABS, rel_l2=ATTN_REL_L2):
    err = float(np.abs(got.astype(np.float64) - want).max())
    ref = float(np.abs(want).max())
    rel = float(np.sqrt(((got.astype(np.float64) - want) ** 2).sum() / (want.astype(np.float64) ** 2).sum()))
    return err <= max_abs * ref and rel <= rel_l2, f"max-abs {err:.3e} (ref max {ref:.3e}, ratio {err / ref:.2e}), rel-L2 {rel:.2e}"


def cpu_twin_of(layer):
    """A CPU-oracle layer holding the very bytes of a device layer (planes, stage, page table): what the oracle then
    computes is attention over the cache the GPU kernels read, whoever wrote it."""
    cpu = orc.CpuLayer(layer.head_dim, layer.kv_heads, layer.pages, layer.table.cpu().numpy(), int(layer.c.sinkhorn_iters))
    cpu.k_code[:] = layer.k_code.cpu().numpy()
    cpu.v_code[:] = layer.v_code.cpu().numpy()
    cpu.k_scale[:] = layer.k_scale.cpu().numpy().view(np.uint16)
    cpu.v_scale[:] = layer.v_scale.cpu().numpy().view(np.uint16)
    cpu.stage[:] = layer.stage.cpu().numpy().view(np.uint16).reshape(cpu.stage.shape)
    return cpu


def host_threads():
    return os.cpu_count() or 1
