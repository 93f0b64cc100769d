"""OutlierAwareLinear: INT8 linear with the LLM.int8 mixed-precision decomposition.

Drop-in for mps_bitsandbytes/nn/outlier_aware.py:18-219: same constructor, buffers
(``weight_int8`` [N, K], ``weight_scales`` [N], ``outlier_indices`` [n], ``outlier_weights``
[N, n], ``bias``), ``from_linear`` (outlier columns = those whose largest |w| exceeds
``threshold`` x the mean |w|; kept in 16 bits and zeroed in the int8 copy) and forward
semantics.  The reference slices x and W by a boolean mask and runs an int8-dequantised
matmul plus a 16-bit outlier matmul (:123-146); here ``mpsbnb_outlier_linear`` builds both
operands with the outlier columns spliced in and runs one tcgen05 GEMM over the full K.
"""
import ctypes as C

import torch
from torch import Tensor, nn

from .. import _native as N
from ..functional import _FLOAT_DTYPES, _workspace, quantize_rowwise


class OutlierAwareLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, threshold: float = 6.0,
                 compute_dtype=torch.float16, device=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.threshold = threshold
        self.compute_dtype = compute_dtype
        self.register_buffer("weight_int8", torch.zeros(out_features, in_features, dtype=torch.int8, device=device))
        self.register_buffer("weight_scales", torch.ones(out_features, dtype=torch.float32, device=device))
        self.register_buffer("outlier_indices", torch.tensor([], dtype=torch.long, device=device))
        self.register_buffer("outlier_weights", torch.zeros(out_features, 0, dtype=compute_dtype, device=device))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=compute_dtype, device=device))
        else:
            self.register_buffer("bias", None)

    def forward(self, x: Tensor) -> Tensor:
        """outlier_aware.py:84-146.  Output dtype is ``compute_dtype``."""
        N.require_cuda(x, self.weight_int8)
        if self.compute_dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"compute_dtype must be float16 or bfloat16, got {self.compute_dtype}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in _FLOAT_DTYPES:
            x2 = x2.float()
        x2 = x2.contiguous()
        m, n, k = x2.shape[0], self.out_features, self.in_features
        idx = self.outlier_indices.to(torch.long).contiguous()
        ow = self.outlier_weights.to(self.compute_dtype).contiguous()
        bias = None if self.bias is None else self.bias.to(self.compute_dtype).contiguous()
        y = torch.empty(m, n, dtype=self.compute_dtype, device=x2.device)
        lib = N.lib()
        with torch.cuda.device(x2.device):
            ws = _workspace(lib.mpsbnb_outlier_linear_workspace_bytes(N.i64(m), N.i64(n), N.i64(k)), x2.device)
            N.check(lib.mpsbnb_outlier_linear(
                N.ptr(x2), N.dt(x2.dtype), N.i64(m), N.ptr(self.weight_int8.contiguous()),
                N.ptr(self.weight_scales.contiguous()), N.ptr(idx if idx.numel() else None), N.i64(idx.numel()),
                N.ptr(ow if idx.numel() else None), N.i64(n), N.i64(k), N.ptr(bias), N.dt(self.compute_dtype), N.ptr(y),
                N.dt(self.compute_dtype), N.ptr(ws), C.c_size_t(ws.numel()), N.stream()), "outlier_linear")
        return y.view(*lead, n)

    @classmethod
    def from_linear(cls, linear: nn.Linear, threshold: float = 6.0, device=None) -> "OutlierAwareLinear":
        """outlier_aware.py:148-212."""
        if device is None:
            device = linear.weight.device
        dtype = linear.weight.dtype
        if dtype not in (torch.float16, torch.bfloat16):
            dtype = torch.float16
        layer = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, threshold=threshold,
                    compute_dtype=dtype, device=device)
        weight = linear.weight.data.to(device)
        # statistics of the weight as the reference takes them (in the weight's own dtype, :188-190)
        col_max = weight.abs().max(dim=0).values
        mean_abs = weight.abs().mean()
        outlier_indices = torch.where(col_max > (threshold * mean_abs))[0]
        if len(outlier_indices) > 0:
            layer.outlier_indices = outlier_indices
            layer.outlier_weights = weight[:, outlier_indices].to(dtype)
            weight_for_int8 = weight.clone()
            weight_for_int8[:, outlier_indices] = 0
        else:
            weight_for_int8 = weight
        q, s = quantize_rowwise(weight_for_int8)
        layer.weight_int8.copy_(q)
        layer.weight_scales.copy_(s)
        if linear.bias is not None:
            layer.bias.copy_(linear.bias.data.to(dtype))
        return layer

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"threshold={self.threshold}, outliers={len(self.outlier_indices)}")
