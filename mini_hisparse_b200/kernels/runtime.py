"""The runtime of each compute dtype: which kernel a part's matrix product runs on.

float32: the CUDA-core product (true 32-bit: FFMA, no tensor core, no reduced-precision mode).
bfloat16: the tcgen05 tensor-core product; with few tokens the weights stream through the
128-row operand and the K range is split over enough CTAs to fill the GPU (the consumer sums
the partial matrices in order).  Shapes the tensor-core kernel refuses (K or a row stride not a
multiple of 8) go to the CUDA-core product, which takes any shape.
"""
from __future__ import annotations

import torch

from ..parts.base import Product, Runtime, Workspace
from . import api as K

BK = 64            # K elements per pipeline stage of the tensor-core kernel
MIN_KB_PER_SPLIT = 4


class Float32Runtime(Runtime):
    def kernel_modules(self):
        return ("elementwise", "gemm_simt", "attention_simt", "sampling")


class BFloat16Runtime(Runtime):
    def __init__(self, device, dtype=torch.bfloat16):
        super().__init__(device, dtype)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status = None      # set by the runner: kernels report bounded waits that ran out

    def kernel_modules(self):
        return ("elementwise", "gemm_simt", "gemm_tc", "attention_simt", "attention_mma", "sampling")

    def _splits(self, tiles: int, total_kb: int) -> int:
        """Enough K splits for about two CTAs per SM, none empty, none shorter than 4 K blocks."""
        want = min((2 * self.sm_count) // max(tiles, 1), total_kb // MIN_KB_PER_SPLIT)
        if want <= 1:
            return 1
        kb_per = -(-total_kb // want)
        return -(-total_kb // kb_per)

    def linear(self, x, weight, ws: Workspace, name: str, out_dtype=None, bias=None,
               allow_split: bool = True) -> Product:
        M, Kd = x.shape
        N = weight.shape[0]
        out_dtype = out_dtype or self.dtype
        tc_ok = (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and bias is None
                 and Kd % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)
        if not tc_ok:
            out = ws.get(name, (M, N), out_dtype)
            K.gemm_simt(x, weight, out, bias=bias)
            return Product(out)
        total_kb = -(-Kd // BK)
        if M <= 64:
            swap, bn = True, (16 if M <= 16 else 32 if M <= 32 else 64)
            tiles = -(-N // 128)
        else:
            swap = False
            bn = 256 if -(-M // 128) * -(-N // 256) >= self.sm_count or N >= 8192 else 128
            tiles = -(-M // 128) * -(-N // bn)
        nsplit = self._splits(tiles, total_kb) if allow_split else 1
        if nsplit > 1:
            out = ws.get(name, (nsplit, M, N), torch.float32)
            K.gemm_tc(x, weight, out, swap=swap, bn=bn, nsplit=nsplit, split_stride=out.stride(0),
                      status=self.status)
            return Product(out, nsplit)
        out = ws.get(name, (M, N), out_dtype)
        K.gemm_tc(x, weight, out, swap=swap, bn=bn, status=self.status)
        return Product(out)


def make_runtime(device, dtype: torch.dtype) -> Runtime:
    if dtype == torch.float32:
        return Float32Runtime(device, dtype)
    return BFloat16Runtime(device, dtype)
