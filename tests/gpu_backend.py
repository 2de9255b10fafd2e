"""The CUDA library behind the parity-pipeline backend interface (see tests/parity.py).
Every call goes through the C ABI via riemannengine_b200.ops."""
from __future__ import annotations

import numpy as np
import torch

from riemannengine_b200 import capi, ops


class KMapResult(tuple):
    """(offset_ptr, in_idx, out_idx) numpy triple that also carries the device neighbour table."""
    nbr: torch.Tensor
    n_in: int


def dev_coords(c: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(c, np.int32)).cuda()


class GpuBackend:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype

    def insert_and_map(self, coords):
        t = ops.table_build(dev_coords(coords))
        return t.mapping.cpu().numpy(), t.inverse.cpu().numpy()

    def stride_map(self, coords, out_stride):
        aligned = ops.coords_stride(dev_coords(coords), out_stride)
        t = ops.table_build(aligned)
        return t.coords.cpu().numpy(), t.inverse.cpu().numpy()

    def region_offsets(self, ksize, dilation, tensor_stride):
        return ops.region_offsets(capi.HYPER_CUBE, ksize, dilation, tensor_stride)

    def conv_kernel_map(self, in_coords, out_coords, offsets, transposed=False):
        table = ops.table_build(dev_coords(in_coords))
        assert table.n_unique == len(in_coords)
        res = ops.kmap_build(table, dev_coords(out_coords), -offsets if transposed else offsets)
        ptr, a, q = res.pairs()
        out = KMapResult((ptr.numpy(), a.cpu().numpy(), q.cpu().numpy()))
        out.nbr, out.n_in = res.nbr, len(in_coords)
        return out

    def _t(self, a):
        return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda().to(self.dtype)

    def conv_forward(self, feats, weights, kmap, n_in, n_out):
        y = ops.conv_forward(self._t(feats), self._t(weights), kmap.nbr)
        return y.float().cpu().numpy()

    def conv_backward(self, feats, grad_out, weights, kmap, n_in, n_out):
        nbr_t = ops.kmap_transpose(kmap.nbr, n_in)
        g = self._t(grad_out)
        gi = ops.conv_backward_input(g, self._t(weights), nbr_t)
        gw = ops.conv_backward_weight(self._t(feats), g, kmap.nbr)
        return gi.float().cpu().numpy(), gw.cpu().numpy()
