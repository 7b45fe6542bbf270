"""y = x W^T for a weight stored as in the checkpoint, [out, in].

The reference transposes every projection at load (runtime/LLM.h:146-156) for its
K x N kernels; the kernels here read [out, in] directly, which is already K-major
for both operands, so nothing is repacked.  Float32 always runs on the CUDA cores
with float32 accumulation (no tensor-core mode); bfloat16 runs on the tcgen05 kernel
where the shape allows it and on the same CUDA-core kernel otherwise.
"""
from __future__ import annotations

import torch

from ..csrc import ops


# Whether the built-in parts hand split-K partial results to the next kernel instead of summing
# them with a kernel of their own.  Measured on B200 at batch 8: 54.7 us per layer with the
# consumers summing (four splits' loads in flight at a time) against 56.8 us with reduction kernels.
FUSE_PARTIALS = True


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int, allow_partial: bool = False,
           bias: torch.Tensor = None, cta_limit: int = 0):
    """out[:rows] = x[:rows] @ weight.T (+ bias, float32 [out features]); out may be float32 for
    bfloat16 inputs.  cta_limit > 0 keeps a product of few rows to so many CTAs (it then leaves SMs
    to the kernel after it).  With a bias the product is summed into `out` and the bias added there by a
    kernel of its own (the reference adds it in the product's epilogue, model/modules/Linear.h:12-34).

    With allow_partial the result may come back as an ops.PartialSum (a split-K product whose
    partial results are still to be summed) instead of in `out`: pass it straight to a kernel
    that takes one (add_rmsnorm, silu_mul, rope_kv_write, gather_rows), before any other product."""
    if rows == 0:
        return out
    if bias is not None:
        allow_partial = False
    if x.dtype == torch.bfloat16 and ops.gemm_fast_available(x, weight, out, rows):
        res = ops.gemm_fast(x, weight, out, rows, allow_partial=allow_partial, cta_limit=cta_limit)
    else:
        ops.gemm_simt(x, weight, out, rows)
        res = out
    if bias is not None:
        ops.add_bias(out, bias, rows)
    return res


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """out[:rows] = silu(x @ gate.T) * (x @ up.T) for weight = [gate; up] stacked along its rows,
    with the activation applied in the product's epilogue.  Returns False, having done nothing,
    where that is not possible (float32, shapes the tensor-core kernel refuses, or so few rows
    that the product splits its K dimension): the caller then runs the product and the activation
    kernel."""
    if rows == 0:
        return True
    if x.dtype != torch.bfloat16 or not ops.gemm_swiglu_available(x, weight, out, rows):
        return False
    ops.gemm_swiglu(x, weight, out, rows)
    return True
