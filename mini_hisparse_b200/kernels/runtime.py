"""The runtime of each compute dtype: which kernel a part's matrix product runs on.

float32: the CUDA-core product (true 32-bit: FFMA, no tensor core, no reduced-precision mode).
bfloat16: the tcgen05 tensor-core product; with up to 64 tokens the weights stream through the
128-row operand and the K range is split over enough CTAs to fill the GPU (the consumer sums
the partial matrices in order); with more, a persistent kernel gives every SM the same share
of (tile, K block) units.  Shapes the tensor-core kernel refuses (K or a row stride not a
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
        return ("elementwise", "gemm_simt", "sampling")


class BFloat16Runtime(Runtime):
    def __init__(self, device, dtype=torch.bfloat16):
        super().__init__(device, dtype)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status = None      # set by the runner: kernels report bounded waits that ran out
        self._scratch = None    # workspace of the persistent product, made at its first use

    def scratch(self):
        if self._scratch is None:
            self._scratch = K.stream_k_scratch(self.device)
        return self._scratch

    def kernel_modules(self):
        return ("elementwise", "gemm_simt", "gemm_tc", "sampling")

    def _splits(self, tiles: int, total_kb: int) -> int:
        """Enough K splits for about two CTAs per SM, none empty, none shorter than 4 K blocks."""
        want = min((2 * self.sm_count) // max(tiles, 1), total_kb // MIN_KB_PER_SPLIT)
        if want <= 1:
            return 1
        kb_per = -(-total_kb // want)
        return -(-total_kb // kb_per)

    GATE_BLOCK = 16     # gate and up rows are interleaved in blocks of this many rows

    def swiglu_layout(self, gate: torch.Tensor, up: torch.Tensor):
        """The stacked gate/up weight in the layout this runtime's SwiGLU product wants, and the
        block size of that layout (the rows of a block of gate are followed by the same rows of up)."""
        I, Kd = gate.shape
        if I % self.GATE_BLOCK or Kd % 8:
            return torch.cat((gate, up), 0).contiguous(), I
        b = self.GATE_BLOCK
        w = torch.stack((gate.view(I // b, b, Kd), up.view(I // b, b, Kd)), 1).reshape(2 * I, Kd)
        return w.contiguous(), b

    def linear_swiglu(self, x, weight, block: int, ws: Workspace, name: str) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for a weight from swiglu_layout(): fused into the product's
        epilogue when the layout is interleaved, else the product followed by the gate kernel."""
        M, Kd = x.shape
        I = weight.shape[0] // 2
        out = ws.get(name, (M, I), self.dtype)
        if block == self.GATE_BLOCK and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0:
            if M <= 64:
                K.gemm_tc_swiglu(x, weight, out, swap=True, bn=(16 if M <= 16 else 32 if M <= 32 else 64),
                                 status=self.status)
            else:
                K.gemm_tc_swiglu(x, weight, out, swap=False, bn=0, status=self.status, scratch=self.scratch())
            return out
        gu = self.linear(x, weight, ws, name + "_gu")
        K.swiglu(gu.tensor, out, nsplit=gu.nsplit, split_stride=gu.split_stride, block=block)
        return out

    def qkv_rope_append(self, x, weight, bias, ctx, position, block_table, q_out, cache_storage, *,
                        nq, nkv, d, page_size, write_kv) -> bool:
        """More than 64 tokens and head size 64 or 128: the persistent product's epilogue rotates and
        appends, so the float32 q/k/v matrix is never written (a third of that product's time in a
        2,048-token prefill went into writing and re-reading it)."""
        M, Kd = x.shape
        rdim = int(getattr(position, "rotary_dim", 0) or 0)
        interleaved = bool(getattr(position, "interleaved", False))
        if (M <= 64 or not K.gemm_tc_qkv_rope_supports(d, rdim, interleaved) or x.dtype != torch.bfloat16
                or weight.dtype != torch.bfloat16
                or cache_storage.dtype != torch.bfloat16 or Kd % 8 or x.stride(0) % 8 or weight.stride(0) % 8
                or x.data_ptr() % 16 or weight.data_ptr() % 16 or not cache_storage.is_contiguous()):
            return False
        table = None
        if rdim:
            tables = ctx.extras.setdefault("rope_tables", {})
            key = position.spec            # frozen dataclass: layers with the same encoding share the table
            table = tables.get(key)
            if table is None:              # once per step for all layers with this encoding
                table = ctx.ws.get(f"rope_table_{len(tables)}", (M, rdim), torch.float32)
                K.rope_table(ctx.positions, position.inv_freq, table)
                tables[key] = table
        K.gemm_tc_qkv_rope(x, weight, bias, table, ctx.positions, ctx.tok_seg, block_table, q_out, cache_storage,
                           nq=nq, nkv=nkv, d=d, page_size=page_size, rotary_dim=rdim, interleaved=interleaved,
                           write_kv=write_kv, status=self.status)
        return True

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
        tiles256 = -(-M // 128) * -(-N // 256)
        if M > 64 and (2 * tiles256 >= self.sm_count or not allow_split):
            # the persistent kernel: tiles of 128 tokens x 256, its CTAs share the last tiles' K range
            out = ws.get(name, (M, N), out_dtype)
            K.gemm_tc(x, weight, out, swap=False, bn=0, status=self.status, scratch=self.scratch())
            return Product(out)
        if M <= 64:
            swap, bn = True, (16 if M <= 16 else 32 if M <= 32 else 64)
            nsplit = self._splits(-(-N // 128), total_kb) if allow_split else 1
        else:
            # too few tiles for the SMs: cut K so that one round of CTAs covers them; up to 256
            # tokens ride as the narrow operand of one tile
            swap = M <= 256
            bn = 128 if M <= 128 else 256
            tiles = -(-N // 128) if swap else tiles256
            nsplit = max(1, min(self.sm_count // tiles, total_kb // MIN_KB_PER_SPLIT))
            kb_per = -(-total_kb // nsplit)
            nsplit = -(-total_kb // kb_per)
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
